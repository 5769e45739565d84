"""GPU: FP8 GEMM through the C ABI.  Small and ragged shapes against the CPU oracle (same codes in), the
full 4096^3 configuration against the order-exact SIMT kernel and size-independent properties.

Tolerance (stated by the task): max relative error <= 1e-2 after dequantization, bf16 output.  Relative
error is |got - ref| / max(|ref|, tau) with tau = 1e-3 * rms(ref), so that near-zero outputs do not divide
by zero; the un-floored count is asserted too."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def rel_err(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    tau = 1e-3 * np.sqrt((ref ** 2).mean()) + 1e-30
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), tau)).max())


def _quantize(oracle, x, rows, cols, mode):
    codes, scales, bad = oracle.fp8_quantize_rows(x, rows, cols, 0, mode)
    assert bad == -1
    return codes.reshape(rows, cols), scales


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 128, 256), (256, 512, 1024), (64, 64, 64), (100, 200, 304),
                                   (129, 257, 144), (384, 1000, 512), (1000, 136, 2048), (8, 512, 256), (300, 300, 100),
                                   (1, 4096, 4096), (3, 130, 192), (17, 1000, 8192), (32, 256, 320), (12, 64, 64), (40, 200, 128)])
def test_gemm_fp8_vs_oracle(cuda, oracle, M, N, K):
    from oxicuda_b200.blas import gemm_fp8
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    for mode in (0, 1):                           # reference codec codes, RNE codes
        ac, sa = _quantize(oracle, a, 1, M * K, mode)       # per-tensor scales (config 2)
        wc, sw = _quantize(oracle, w, 1, N * K, mode)
        ac, wc = ac.reshape(M, K), wc.reshape(N, K)
        # the tensor core decodes IEEE-style; the oracle in decode mode 1 does the same
        ref = oracle.gemm_fp8(ac, wc, sa, sw, 0, 1, "bf16")
        got = gemm_fp8(_t(ac, cuda), _t(wc, cuda), _t(sa, cuda), _t(sw, cuda)).float().cpu().numpy()
        assert rel_err(got, ref) <= TOL, (M, N, K, mode)
        if mode == 0:
            # the reference's own composition (its codec's encode AND decode, then the f32 matmul): its decoder
            # reads subnormal codes as 2^-6*(1+m/8), which the code rewrite reproduces on the tensor core
            from oxicuda_b200.quant import Fp8Codec
            codec = Fp8Codec.e4m3("ref")
            ref0 = oracle.gemm_fp8(ac, wc, sa, sw, 0, 0, "bf16")
            got0 = gemm_fp8(codec.to_reference_decode_codes(_t(ac, cuda)), codec.to_reference_decode_codes(_t(wc, cuda)),
                            _t(sa, cuda), _t(sw, cuda)).float().cpu().numpy()
            assert rel_err(got0, ref0) <= TOL, (M, N, K, mode)
        # f32 output, per-row (per-token x per-channel) scales
        sa_r = (rng.random(M).astype(np.float32) + 0.5) * sa[0]
        sw_r = (rng.random(N).astype(np.float32) + 0.5) * sw[0]
        ref = oracle.gemm_fp8(ac, wc, sa_r, sw_r, 0, 1, "f32")
        got = gemm_fp8(_t(ac, cuda), _t(wc, cuda), _t(sa_r, cuda), _t(sw_r, cuda), out_dtype=torch.float32).cpu().numpy()
        assert rel_err(got, ref) <= 1e-3, (M, N, K, mode)   # fp32 out: only the tensor core's accumulation differs


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (7, 1000, 1024), (16, 4096, 4096), (17, 300, 256), (33, 640, 2048),
                                   (64, 2304, 1024), (100, 520, 384), (128, 1024, 512), (4, 19000, 256), (2, 40000, 128)])
def test_weight_stationary_tcgen05_kernel(cuda, oracle, M, N, K, switches):
    """The few-token kernel (weights as the M = 128 operand), forced on: one tile per CTA, several tiles per CTA
    (19000 and 40000 rows), the even split with partial sums (few rows, long K), ragged last tiles, every token padding."""
    from oxicuda_b200.blas import gemm_fp8
    switches(B2Q_FP8_SKINNY=1)
    rng = np.random.default_rng(M * 11 + N * 5 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    ac, sa = _quantize(oracle, a, 1, M * K, 1)
    wc, sw = _quantize(oracle, w, 1, N * K, 1)
    ac, wc = ac.reshape(M, K), wc.reshape(N, K)
    ref = oracle.gemm_fp8(ac, wc, sa, sw, 0, 1, "bf16")
    got = gemm_fp8(_t(ac, cuda), _t(wc, cuda), _t(sa, cuda), _t(sw, cuda)).float().cpu().numpy()
    assert rel_err(got, ref) <= TOL
    sa_r = (rng.random(M).astype(np.float32) + 0.5) * sa[0]
    sw_r = (rng.random(N).astype(np.float32) + 0.5) * sw[0]
    ref = oracle.gemm_fp8(ac, wc, sa_r, sw_r, 0, 1, "f32")
    for _ in range(3):                                # back to back: launches overlap their tails
        got = gemm_fp8(_t(ac, cuda), _t(wc, cuda), _t(sa_r, cuda), _t(sw_r, cuda), out_dtype=torch.float32)
    from oxicuda_b200._lib import default_handle
    default_handle().check()
    assert rel_err(got.cpu().numpy(), ref) <= 1e-3


def test_weights_written_right_before_the_call(cuda, oracle, switches):
    """With static_weights off the few-token kernel reads nothing before the previous kernel of the stream (here the
    one that produces the weight codes) has completed."""
    from oxicuda_b200.blas import gemm_fp8
    from oxicuda_b200.quant import Fp8Codec
    from oxicuda_b200._lib import default_handle
    switches(B2Q_FP8_SKINNY=1)
    h = default_handle()
    h.set_static_weights(False)
    try:
        M, N, K = 8, 8192, 4096
        codec = Fp8Codec.e4m3("rne")
        g = torch.Generator(device=cuda).manual_seed(5)
        a = torch.randn(M, K, device=cuda, generator=g)
        ac, sa = codec.quantize_rows(a, 1, M * K)
        for rep in range(5):
            w = torch.randn(N, K, device=cuda, generator=g) * 0.02
            wc, sw = codec.quantize_rows(w, 1, N * K)            # kernels on the same stream, no synchronisation
            got = gemm_fp8(ac.view(M, K), wc.view(N, K), sa, sw, out_dtype=torch.float32)
            ref = oracle.gemm_fp8(ac.view(M, K).cpu().numpy(), wc.view(N, K).cpu().numpy(), sa.cpu().numpy(), sw.cpu().numpy(), 0, 1, "f32")
            assert rel_err(got.cpu().numpy(), ref) <= 1e-3, rep
    finally:
        h.set_static_weights(True)


def test_simt_kernel_reproduces_oracle_order(cuda, oracle):
    """The checker kernel (software decode, k-ascending fp32 FMA) equals the oracle to the last bit."""
    from oxicuda_b200.blas import gemm_fp8
    rng = np.random.default_rng(31)
    M, N, K = 96, 80, 520
    ac = rng.integers(0, 256, (M, K)).astype(np.uint8)
    wc = rng.integers(0, 256, (N, K)).astype(np.uint8)
    ac[(ac & 0x7F) == 0x7F] = 0x3C
    wc[(wc & 0x7F) == 0x7F] = 0x3C                # no NaN codes
    sa = np.array([0.013], np.float32)
    sw = rng.random(N).astype(np.float32)
    for decode, mode in (("ref", 0), ("ieee", 1)):
        ref = oracle.gemm_fp8(ac, wc, sa, sw, 0, mode, "f32")
        got = gemm_fp8(_t(ac, cuda), _t(wc, cuda), _t(sa, cuda), _t(sw, cuda), out_dtype=torch.float32, simt_decode=decode)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32)), decode


def test_every_code_pair_is_exact_on_the_tensor_core(cuda, oracle):
    """One product per output: A holds every E4M3 code on the diagonal positions, so out[m,n] = a_m * w_n
    exactly (a single non-zero term); all 254x254 finite pairs must match the IEEE decode product."""
    from oxicuda_b200.blas import gemm_fp8
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)     # 254 finite codes
    n = codes.size
    K = 256
    a = np.zeros((n, K), np.uint8)
    w = np.zeros((n, K), np.uint8)
    a[:, 5] = codes
    w[:, 5] = codes
    one = np.ones(1, np.float32)
    got = gemm_fp8(_t(a, cuda), _t(w, cuda), _t(one, cuda), _t(one, cuda), out_dtype=torch.float32).cpu().numpy()
    vals = oracle.fp8_decode(codes, 0, 1).astype(np.float32)
    assert np.array_equal(got, np.outer(vals, vals).astype(np.float32))


def test_config2_full_size_4096(cuda, oracle):
    """A ~N(0,1), B ~N(0,0.02) at 4096^3, per-tensor absmax scales, bf16 out."""
    from oxicuda_b200.blas import gemm_fp8
    from oxicuda_b200.quant import Fp8Codec
    M = N = K = 4096
    g = torch.Generator(device=cuda).manual_seed(0xB2000001)
    a = torch.randn(M, K, device=cuda, generator=g)
    w = torch.randn(N, K, device=cuda, generator=g) * 0.02
    for rounding, mode in (("ref", 0), ("rne", 1)):
        codec = Fp8Codec.e4m3(rounding)
        ac, sa = codec.quantize_rows(a, 1, M * K)
        wc, sw = codec.quantize_rows(w, 1, N * K)
        ac, wc = ac.view(M, K), wc.view(N, K)
        out = gemm_fp8(ac, wc, sa, sw)
        # (1) codes and scales are bit-exact with the oracle on a slice the CPU finishes quickly
        sl = slice(0, 64)
        c_ref, s_ref, _ = oracle.fp8_quantize_rows(a.cpu().numpy(), 1, M * K, 0, mode)
        assert np.array_equal(sa.cpu().numpy(), s_ref) and np.array_equal(ac.cpu().numpy().reshape(-1), c_ref)
        # (2) rows/columns sampled across all tiles against the oracle GEMM on the same codes
        rows = np.r_[0:16, 2040:2056, 4080:4096]
        ref = oracle.gemm_fp8(ac[rows].cpu().numpy(), wc.cpu().numpy(), sa.cpu().numpy(), sw.cpu().numpy(), 0, 1, "bf16")
        assert rel_err(out[rows].float().cpu().numpy(), ref) <= TOL
        # (3) whole output against the order-exact SIMT kernel
        chk = gemm_fp8(ac, wc, sa, sw, simt_decode="ieee")
        tau = 1e-3 * chk.float().pow(2).mean().sqrt()
        err = ((out.float() - chk.float()).abs() / chk.float().abs().clamp_min(tau)).max().item()
        assert err <= TOL, err
        # (4) linearity in the scales: doubling a scale doubles every output exactly (power of two)
        out2 = gemm_fp8(ac, wc, sa * 2, sw)
        assert torch.equal(out2.float(), out.float() * 2)
        # (5) row permutation of A permutes the rows of the output bit for bit
        perm = torch.randperm(M, device=cuda, generator=g)
        assert torch.equal(gemm_fp8(ac[perm].contiguous(), wc, sa, sw), out[perm])


def test_gemm_fp8_validation_order(cuda):
    from oxicuda_b200 import _lib
    from oxicuda_b200.blas import gemm_fp8
    one = torch.ones(1, device=cuda)
    z = lambda *s: torch.zeros(*s, dtype=torch.uint8, device=cuda)
    with pytest.raises(_lib.InvalidDimension):                       # zero dims first (gemm_api.rs:142-146)
        gemm_fp8(z(0, 64), z(64, 64), one, one)
    with pytest.raises(_lib.DimensionMismatch):                      # inner mismatch (gemm_api.rs:149-153)
        gemm_fp8(z(64, 64), z(64, 128), one, one)
    buf = z(64 * 64 * 4)
    with pytest.raises(_lib.InvalidArgument):                        # C overlaps A (gemm_api.rs:189-195)
        gemm_fp8(buf[:4096].view(64, 64), z(64, 64), one, one, out=buf[:8192].view(torch.bfloat16).view(64, 64))
    with pytest.raises(_lib.DimensionMismatch):
        gemm_fp8(z(64, 64), z(64, 64), torch.ones(3, device=cuda), one)


@pytest.mark.parametrize("M,N,K", [(384, 512, 512), (128, 384, 256), (300, 200, 128), (8, 4096, 4096), (48, 256, 512)])
def test_epilogue_ops_alpha_beta_bias_and_kn_layout(cuda, oracle, M, N, K):
    """b2q_gemm_fp8_ex against the reference's epilogue statement (epilogue.rs:99-196) applied to the oracle's f32 GEMM:
    every EpilogueOp, alpha / beta with C in place, bf16 and f32 outputs, the fused store path of the prefill kernels
    (first three shapes), the elementwise pass behind the few-token kernels (last two), and the [K x N] operand."""
    from oxicuda_b200.blas import EpilogueOp, gemm_fp8_ex
    from oxicuda_b200.quant import Fp8Codec
    rng = np.random.default_rng(M + N + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    codec = Fp8Codec.e4m3("rne")
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(cuda)
    ac, sa = codec.quantize_rows(t(a), M, K)
    wc, sw = codec.quantize_rows(t(w), N, K)
    ac, wc = ac.view(M, K), wc.view(N, K)
    plain = np.asarray(oracle.gemm_fp8(ac.cpu().numpy(), wc.cpu().numpy(), sa.cpu().numpy(), sw.cpu().numpy(), 0, 1, "f32"), np.float64).reshape(M, N)
    bias = rng.standard_normal(N).astype(np.float32)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    gelu = lambda v: v / (1.0 + np.exp2(-1.702 * 1.4426950408889634 * v))

    def check(got, ref, tol=1e-2):
        rms = np.sqrt((ref ** 2).mean()) + 1e-30
        assert float((np.abs(got.double().cpu().numpy() - ref) / (np.abs(ref) + rms)).max()) <= tol

    cases = [(EpilogueOp.LinearCombination, 0.5, 0.0, None, lambda v: v),
             (EpilogueOp.LinearCombination, 2.0, -0.75, None, lambda v: v),
             (EpilogueOp.LinearCombinationRelu, 1.0, 0.0, None, lambda v: np.maximum(v, 0)),
             (EpilogueOp.LinearCombinationGelu, 1.0, 0.0, None, gelu),
             (EpilogueOp.LinearCombinationBias, 1.0, 0.0, bias, lambda v: v),
             (EpilogueOp.LinearCombinationBiasRelu, 1.5, 0.25, bias, lambda v: np.maximum(v, 0))]
    for dtype in (torch.bfloat16, torch.float32):
        for op, alpha, beta, b, act in cases:
            c_dev = t(c0).to(dtype)
            c_host = c_dev.double().cpu().numpy()
            ref = alpha * plain + beta * c_host + (b.astype(np.float64)[None, :] if b is not None else 0.0)
            ref = act(ref)
            got = gemm_fp8_ex(ac, wc, sa, sw, out=c_dev, alpha=alpha, beta=beta, bias=t(b) if b is not None else None, epilogue=op)
            check(got, ref)
    # the reference's [K x N] operand B
    wkn = wc.t().contiguous()
    got = gemm_fp8_ex(ac, wkn, sa, sw, w_is_kn=True, out_dtype=torch.float32)
    check(got, plain, 2e-3)
    with pytest.raises(Exception):
        gemm_fp8_ex(ac, wc, sa, sw, epilogue=EpilogueOp.LinearCombinationBias)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(512, 1024, 512), (300, 512, 256), (48, 512, 512), (4096, 2048, 1024), (2560, 2048, 256), (2304, 2304 * 2, 128)])
def test_epilogue_swiglu_pairs(cuda, oracle, M, N, K):
    """EpilogueOp.SwiGluPairs: the gate | up GEMM over rows interleaved per 128 (b2q_interleave_rows128) writes
    silu(gate) * up [M x N / 2] (SwiGluExpert::forward, crates/oxicuda-moe/src/expert/ffn.rs:208-243; silu of
    crates/oxicuda-lm/src/layer/ffn.rs:25-27) from the epilogue of the two-CTA kernel (M > 128) or after the few-token
    kernels (M = 48); checked against the oracle's f32 GEMM of the gate and of the up rows.  The last two shapes have 80
    and 162 tiles on 74 CTA pairs: their last wave runs as half units of 64 gate + 64 up columns."""
    from oxicuda_b200._lib import default_handle, ptr
    from oxicuda_b200.blas import EpilogueOp, gemm_fp8_ex
    from oxicuda_b200.quant import Fp8Codec
    rng = np.random.default_rng(M + N + K + 3)
    F = N // 2
    a = rng.standard_normal((M, K)).astype(np.float32)
    wg = (rng.standard_normal((F, K)) * 0.08).astype(np.float32)
    wu = (rng.standard_normal((F, K)) * 0.08).astype(np.float32)
    codec = Fp8Codec.e4m3("rne")
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(cuda)
    ac, sa = codec.quantize_rows(t(a), M, K)
    gc, gs = codec.quantize_rows(t(wg), F, K)
    uc, us = codec.quantize_rows(t(wu), F, K)
    ac = ac.view(M, K)
    wc = torch.empty(N, K, dtype=torch.uint8, device=cuda)
    sw = torch.empty(N, dtype=torch.float32, device=cuda)
    h = default_handle()
    h.call("b2q_interleave_rows128", ptr(gc), ptr(uc), F, K, ptr(wc))
    h.call("b2q_interleave_rows128", ptr(gs), ptr(us), F, 4, ptr(sw))
    # the interleaved layout itself: block j of 256 rows = gate rows [128 j, ...) then up rows [128 j, ...)
    exp_codes = torch.stack([gc.view(F // 128, 128, K), uc.view(F // 128, 128, K)], dim=1).reshape(N, K)
    exp_scales = torch.stack([gs.view(F // 128, 128), us.view(F // 128, 128)], dim=1).reshape(N)
    assert torch.equal(wc, exp_codes) and torch.equal(sw, exp_scales)
    f32 = lambda c, s: np.asarray(oracle.gemm_fp8(ac.cpu().numpy(), c.view(F, K).cpu().numpy(), sa.cpu().numpy(), s.cpu().numpy(), 0, 1, "f32"),
                                  np.float64).reshape(M, F)
    g, u = f32(gc, gs), f32(uc, us)
    ref = g / (1.0 + np.exp(-g)) * u
    got = gemm_fp8_ex(ac, wc, sa, sw, epilogue=EpilogueOp.SwiGluPairs)
    h.check()
    assert got.shape == (M, F)
    rms = np.sqrt((ref ** 2).mean()) + 1e-30
    assert float((np.abs(got.double().cpu().numpy() - ref) / (np.abs(ref) + rms)).max()) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("tp,M,N,K", [(2, 512, 384, 256), (4, 1024, 512, 512), (8, 2048, 256, 128), (4, 384, 1024, 1024)])
def test_scatter_gemm_fills_every_owner_slot(cuda, tp, M, N, K):
    """b2q_gemm_fp8_scatter, the GEMM half of the many-token row-parallel boundary, with all tp ranks played one after the
    other on this GPU (the inboxes are plain local buffers; nothing in this kernel waits): after rank r's launch, slot r
    of owner o's inbox holds rows [o M / tp, (o + 1) M / tp) of rank r's partial product, bit for bit what b2q_gemm_fp8
    writes, with the bias on rank 0 only; slots of other ranks stay untouched."""
    import ctypes as C
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.blas import gemm_fp8, gemm_fp8_ex, EpilogueOp
    from oxicuda_b200.quant import Fp8Codec
    g = torch.Generator(device=cuda).manual_seed(tp * 1000 + M)
    codec = Fp8Codec.e4m3("rne")
    rows = M // tp
    inbox = [torch.full((tp, rows, N), -7.0, dtype=torch.bfloat16, device=cuda) for _ in range(tp)]
    ptrs = (C.c_void_p * tp)(*[t.data_ptr() for t in inbox])
    bias = torch.randn(N, device=cuda, generator=g)
    h = L.default_handle()
    want = []
    for r in range(tp):
        ac, sa = codec.quantize_rows(torch.randn(M, K, device=cuda, generator=g), M, K)
        wc, sw = codec.quantize_rows(torch.randn(N, K, device=cuda, generator=g) * 0.05, N, K)
        ac, wc = ac.view(M, K), wc.view(N, K)
        h.call("b2q_gemm_fp8_scatter", L.ptr(ac), L.ptr(wc), M, N, K, L.FP8_E4M3, L.ptr(sa), L.ptr(sw), L.ptr(bias) if r == 0 else None, ptrs, tp, r)
        want.append(gemm_fp8_ex(ac, wc, sa, sw, bias=bias, epilogue=EpilogueOp.LinearCombinationBias) if r == 0 else gemm_fp8(ac, wc, sa, sw))
        h.check()
        for o in range(tp):                                   # slots of ranks that have not run yet are untouched
            for later in range(r + 1, tp):
                assert bool((inbox[o][later] == -7.0).all())
    for r in range(tp):
        for o in range(tp):
            assert torch.equal(inbox[o][r], want[r][o * rows:(o + 1) * rows]), (r, o)
    with pytest.raises(L.UnsupportedOperation):
        h.call("b2q_gemm_fp8_scatter", L.ptr(ac), L.ptr(wc), 100, N, K, L.FP8_E4M3, L.ptr(sa), L.ptr(sw), None, ptrs, tp, 0)
