"""GPU: block-scaled FP4 weight-only decode GEMV through the C ABI against the CPU oracle
(dequantize_fp4 followed by an f32 dot product), bf16 out, max relative error <= 1e-2."""
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


def _case(cuda, oracle, tokens, N, K, scale_mode, seed, out_dtype=torch.bfloat16):
    from oxicuda_b200.blas import gemv_fp4_wo
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(N * K) * 0.02).astype(np.float32)
    codes, scales = oracle.fp4_block_quantize(w, 32, 0, scale_mode)
    x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16)
    xb = x.view(torch.int16).numpy().view(np.uint16)
    ref = oracle.gemv_fp4(codes, scales, xb, tokens, N, K, 32, "bf16" if out_dtype == torch.bfloat16 else "f32")
    got = gemv_fp4_wo(_t(codes, cuda), _t(scales, cuda), x.to(cuda), N, K, out_dtype=out_dtype)
    return rel_err(got.float().cpu().numpy(), ref)


@pytest.mark.parametrize("tokens", [1, 4, 16, 32])
@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_llama3_8b_projections(cuda, oracle, tokens, N, K):
    for scale_mode in (1, 0):                       # E8M0 (the configuration's wording) and f32 (reference) scales
        assert _case(cuda, oracle, tokens, N, K, scale_mode, N + K + tokens) <= TOL


@pytest.mark.parametrize("tokens,N,K", [(1, 16, 128), (3, 100, 256), (7, 17, 640), (9, 2050, 1152), (31, 130, 128), (32, 64, 8192)])
def test_ragged_shapes(cuda, oracle, tokens, N, K):
    for scale_mode in (1, 0):
        assert _case(cuda, oracle, tokens, N, K, scale_mode, 5, torch.float32) <= 2e-3


@pytest.mark.parametrize("tokens,N,K", [(4, 38400, 1024), (1, 28672, 4096), (32, 14336, 4096), (8, 4096, 14336), (5, 13400, 2560)])
def test_tensor_core_block_scaled_path(cuda, oracle, tokens, N, K, switches):
    """The tcgen05 kind::mxf8f6f4 kernel, forced on: several whole tiles per CTA (38400 rows = 300 tiles), one tile
    per CTA, the even split with partial sums (4096 rows), a ragged last tile (13400 rows)."""
    switches(B2Q_GEMV_MX=1)
    assert _case(cuda, oracle, tokens, N, K, 1, 11 * tokens + N, torch.float32) <= 2e-3
    assert _case(cuda, oracle, tokens, N, K, 1, 13 * tokens + N, torch.bfloat16) <= TOL


@pytest.mark.parametrize("tokens,N,K", [(1, 28672, 4096), (3, 4096, 4096), (4, 13400, 2560), (5, 14336, 4096), (16, 4096, 14336), (13, 8192, 1024),
                                        (7, 300, 256)])
def test_dense_format_mxf4_kernel(cuda, oracle, tokens, N, K, switches):
    """The tcgen05 kind::mxf4 kernel (dense 4-bit operands, activations as seven E2M1 terms), forced on: whole tiles and
    the even split with partial sums, the in-kernel activation split (up to 4 tokens) and the pre-pass (5 to 16), ragged
    last tiles.  Seven terms leave under 2^-19 of a block's maximum, so the f32 bound of the other kernels holds."""
    switches(B2Q_GEMV_STREAM=2)
    assert _case(cuda, oracle, tokens, N, K, 1, 17 * tokens + N, torch.float32) <= 2e-3
    assert _case(cuda, oracle, tokens, N, K, 1, 19 * tokens + N, torch.bfloat16) <= TOL


def test_back_to_back_calls_with_different_operands(cuda, oracle, switches):
    """Consecutive launches overlap their tails (programmatic dependent launch): every call must still see its own
    activations, scales and partial sums."""
    from oxicuda_b200.blas import gemv_fp4_wo
    from oxicuda_b200._lib import default_handle
    switches(B2Q_GEMV_MX=1)
    rng = np.random.default_rng(7)
    N, K = 4096, 4096
    sets = []
    for tokens in (1, 8, 32):
        w = (rng.standard_normal(N * K) * 0.02).astype(np.float32)
        codes, scales = oracle.fp4_block_quantize(w, 32, 0, 1)
        x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16)
        xb = x.view(torch.int16).numpy().view(np.uint16)
        ref = np.asarray(oracle.gemv_fp4(codes, scales, xb, tokens, N, K, 32, "f32")).reshape(tokens, N)
        sets.append((_t(codes, cuda), _t(scales, cuda), x.to(cuda), ref))
    outs = []
    for rep in range(30):
        c, s, x, _ = sets[rep % 3]
        outs.append((rep % 3, gemv_fp4_wo(c, s, x, N, K, out_dtype=torch.float32)))
    default_handle().check()
    for i, o in outs:
        assert rel_err(o.cpu().numpy(), sets[i][3]) <= 2e-3


def test_codes_map_exactly(cuda, oracle):
    """x = one-hot rows picks single weights: every E2M1 code times a power-of-two scale is exact."""
    from oxicuda_b200.blas import gemv_fp4_wo
    N, K = 16, 128
    codes = np.zeros((N, K // 2), np.uint8)
    for n in range(N):
        codes[n, :] = n | (n << 4)                  # row n holds code n everywhere
    scales = np.full((N, K // 32), 127 + 3, np.uint8)   # 2^3
    for pos in (0, 1, 37, 127):
        x = torch.zeros(1, K, dtype=torch.bfloat16)
        x[0, pos] = 1.0
        got = gemv_fp4_wo(_t(codes, cuda), _t(scales, cuda), x.to(cuda), N, K, out_dtype=torch.float32).cpu().numpy()[0]
        want = np.array([oracle.fp4_dequantize_one(n, 0) * 8.0 for n in range(N)], np.float32)
        assert np.array_equal(got, want), pos


@pytest.mark.parametrize("tokens", [1, 5, 16, 32])
def test_e8m0_exponents_outside_the_f16_range(cuda, oracle, tokens):
    """Legal MX tensors whose block exponents cannot be folded into f16 codes: 2^20 and 2^14 (code * scale overflows
    f16) take the exact fp32 statement inside the kernel, 2^-40 flushes (at most 2^-24 per code).  No status is raised
    and the result is the oracle's."""
    from oxicuda_b200._lib import default_handle
    from oxicuda_b200.blas import gemv_fp4_wo
    rng = np.random.default_rng(21 + tokens)
    N, K = 272, 2048
    codes = rng.integers(0, 256, (N, K // 2)).astype(np.uint8)
    scales = rng.integers(127 - 9, 127 - 3, (N, K // 32)).astype(np.uint8)
    scales[3, 5] = 127 + 20
    scales[100, 0] = 127 + 14
    scales[271, K // 32 - 1] = 127 + 20
    scales[7, 9] = 127 - 40
    scales[8, :] = 127 - 40                          # a whole row of tiny blocks
    x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16)
    xb = x.view(torch.int16).numpy().view(np.uint16)
    ref = np.asarray(oracle.gemv_fp4(codes.reshape(-1), scales.reshape(-1), xb, tokens, N, K, 32, "f32"), np.float64).reshape(tokens, N)
    got = gemv_fp4_wo(_t(codes.reshape(-1), cuda), _t(scales.reshape(-1), cuda), x.to(cuda), N, K, out_dtype=torch.float32)
    default_handle().check()                         # nothing recorded
    got = got.cpu().numpy().astype(np.float64)
    # per row: rows with a huge block are dominated by it
    for n in range(N):
        scale = np.abs(ref[:, n]).max() + 1e-300
        assert np.abs(got[:, n] - ref[:, n]).max() <= 2e-3 * scale + 1e-3, n      # flushed blocks: < 2^-24 per code


def test_linearity_and_validation(cuda, oracle):
    from oxicuda_b200 import _lib
    from oxicuda_b200.blas import gemv_fp4_wo
    rng = np.random.default_rng(8)
    N, K = 512, 1024
    w = (rng.standard_normal(N * K) * 0.02).astype(np.float32)
    codes, scales = oracle.fp4_block_quantize(w, 32, 0, 1)
    cd, sd = _t(codes, cuda), _t(scales, cuda)
    x = torch.randn(4, K, device=cuda).to(torch.bfloat16)
    y = gemv_fp4_wo(cd, sd, x, N, K, out_dtype=torch.float32)
    y2 = gemv_fp4_wo(cd, sd, (x.float() * 2).to(torch.bfloat16), N, K, out_dtype=torch.float32)
    assert torch.equal(y2, y * 2)                   # scaling activations by 2 is exact
    y1 = gemv_fp4_wo(cd, sd, x[:1].contiguous(), N, K, out_dtype=torch.float32)
    assert torch.allclose(y1, y[:1], rtol=1e-5, atol=1e-6)     # a token's result does not depend on its batch
    with pytest.raises(_lib.UnsupportedOperation):
        gemv_fp4_wo(cd, sd, torch.zeros(33, K, device=cuda, dtype=torch.bfloat16), N, K)
    with pytest.raises(_lib.InvalidDimension):
        gemv_fp4_wo(cd, sd, x, N, 1000)
    with pytest.raises(_lib.InvalidArgument):
        gemv_fp4_wo(cd, sd, x, N, K, block=48)


@pytest.mark.parametrize("tokens,N,K,block", [(64, 512, 1024, 32), (300, 1000, 256, 64), (1000, 136, 2048, 128), (33, 64, 128, 32),
                                              (4096, 1024, 4096, 32)])
def test_prefill_fp4_weight_only_gemm(cuda, oracle, tokens, N, K, block):
    """Token counts above the decode range: weights expanded to bf16, product on tcgen05 (kind::f16)."""
    from oxicuda_b200.blas import Fp4Format, gemm_fp4_wo
    rng = np.random.default_rng(tokens + N + K)
    w = (rng.standard_normal(N * K) * 0.02).astype(np.float32)
    x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16)
    xb = x.view(torch.int16).numpy().view(np.uint16)
    for scale_mode in (1, 0):
        codes, scales = oracle.fp4_block_quantize(w, block, 0, scale_mode)
        ref = oracle.gemv_fp4(codes, scales, xb, tokens, N, K, block, "bf16")
        got = gemm_fp4_wo(_t(codes, cuda), _t(scales, cuda), x.to(cuda), N, K, block=block).float().cpu().numpy()
        if scale_mode == 1 or tokens <= 32:
            assert rel_err(got, ref) <= TOL, (scale_mode, block)          # power-of-two scales expand to bf16 exactly
        else:
            # an f32 scale times a code is rounded to bf16 (8 significant bits) before the tensor-core product: each
            # weight is off by up to 2^-9 relative, which moves an output by about 1e-3 of the output rms whatever its
            # own size; the bound is therefore 1e-2 relative plus 1e-2 of the rms
            rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
            assert float((np.abs(got - ref) / (np.abs(ref) + rms)).max()) <= TOL, (scale_mode, block)
    if tokens <= 300:                                     # INT4 codes share the kernel
        codes, scales = oracle.fp4_block_quantize(w, block, 1, 0)
        deq = oracle.fp4_block_dequantize(codes, scales, N * K, block, 1).reshape(N, K).astype(np.float64)
        ref = x.float().numpy().astype(np.float64) @ deq.T
        got = gemm_fp4_wo(_t(codes, cuda), _t(scales, cuda), x.to(cuda), N, K, block=block, format=Fp4Format.Int4, out_dtype=torch.float32)
        rms = np.sqrt((ref ** 2).mean())
        assert float((np.abs(got.cpu().numpy() - ref) / (np.abs(ref) + rms)).max()) <= TOL


@pytest.mark.parametrize("tokens,N,K", [(128, 256, 128), (200, 300, 512), (64, 1024, 4096), (1000, 520, 1024), (4096, 14336, 4096)])
def test_blockscaled_prefill_gemm(cuda, oracle, tokens, N, K):
    """b2q_gemm_fp4_blockscaled: the weights feed tcgen05 kind::mxf8f6f4.block_scale as stored.  Split activations keep the
    weight-only result (<= 1e-2, f32 out 2e-3); MX E4M3 activations match the oracle composed with the same activation
    quantizer (restated here in numpy over the oracle's E4M3 codec).  The largest case is a stated prefill shape and is
    checked on a sample of rows."""
    from oxicuda_b200.blas import MicroScalingConfig, MicroScalingQuantizer, ScalingFormat, gemm_fp4_blockscaled
    big = tokens * N * K > 2e10
    g = torch.Generator(device=cuda).manual_seed(tokens + N + K)
    w = torch.randn(N * K, device=cuda, generator=g) * 0.02
    codes, scales = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0)).quantize_fp4(w)
    x = torch.randn(tokens, K, device=cuda, generator=g).to(torch.bfloat16)
    rows = np.arange(0, tokens, max(1, tokens // 48))[:48] if big else np.arange(tokens)
    xs = x[torch.from_numpy(rows).to(cuda)].cpu()
    xb = xs.view(torch.int16).numpy().view(np.uint16)
    cn, sn = codes.cpu().numpy(), scales.cpu().numpy()
    ref = np.asarray(oracle.gemv_fp4(cn, sn, xb, rows.size, N, K, 32, "f32"), np.float64).reshape(rows.size, N)
    got = gemm_fp4_blockscaled(codes, scales, x, N, K, out_dtype=torch.float32)[torch.from_numpy(rows).to(cuda)].cpu().numpy()
    assert rel_err(got, ref) <= 2e-3
    got16 = gemm_fp4_blockscaled(codes, scales, x, N, K)[torch.from_numpy(rows).to(cuda)].float().cpu().numpy()
    assert rel_err(got16, _t(ref.astype(np.float32), "cpu").to(torch.bfloat16).float().numpy()) <= TOL
    # W4A8: one E4M3 code per activation under the block's power-of-two scale (smallest 2^e with max / 2^e <= 448)
    xf = xs.float().numpy().reshape(rows.size, K // 32, 32)
    amax = np.abs(xf).max(axis=2, keepdims=True)
    e = np.where(amax > 0, np.ceil(np.log2(np.maximum(amax, 1e-38) / 448.0)), 0.0)
    e = np.maximum(e, -127.0)
    q = oracle.fp8_decode(oracle.fp8_encode((xf / np.exp2(e)).astype(np.float32).reshape(-1), 0, 1)[0], 0, 1).reshape(xf.shape) * np.exp2(e)
    xq = torch.from_numpy(q.reshape(rows.size, K).astype(np.float32)).to(torch.bfloat16)     # exact: four significant bits
    assert np.array_equal(xq.float().numpy(), q.reshape(rows.size, K).astype(np.float32))
    ref8 = np.asarray(oracle.gemv_fp4(cn, sn, xq.view(torch.int16).numpy().view(np.uint16), rows.size, N, K, 32, "f32"), np.float64).reshape(rows.size, N)
    got8 = gemm_fp4_blockscaled(codes, scales, x, N, K, mxfp8_activations=True, out_dtype=torch.float32)[torch.from_numpy(rows).to(cuda)].cpu().numpy()
    assert rel_err(got8, ref8) <= 2e-3
