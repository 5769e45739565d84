"""GPU: the KV-cache quantizers (bit-exact against the CPU oracle and the reference's own test cases) and the fused
RMSNorm -> FP8 quantizer (against the oracle's RMSNorm + per-token FP8 rule), all through the C ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def _kv_input(rng, n_tokens, head_dim, bf16):
    x = (rng.standard_normal((n_tokens, head_dim)) * rng.uniform(0.05, 4.0, (n_tokens, 1))).astype(np.float32)
    x[:, head_dim // 3] += 11.0                      # an outlier channel, as rotary keys have
    if n_tokens > 2:
        x[1, :] = 0.75                               # a constant row: degenerate range
    if bf16:
        x = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    return x


@pytest.mark.parametrize("bf16", [False, True])
def test_kv_cache_quantizer_bit_exact(cuda, oracle, bf16):
    from oxicuda_b200.kv_cache import KvAxis, KvCacheConfig, KvCacheQuantizer
    rng = np.random.default_rng(21)
    for n_tokens, head_dim in ((1, 1), (12, 16), (16, 8), (10, 12), (257, 128), (1000, 80), (4096, 128), (33, 1030), (70000, 64)):
        x = _kv_input(rng, n_tokens, head_dim, bf16)
        xt = _t(x, cuda).to(torch.bfloat16) if bf16 else _t(x, cuda)
        for axis in (KvAxis.PerToken, KvAxis.PerChannel):
            for bits in (8, 4, 2):
                cache = KvCacheQuantizer(KvCacheConfig.new(bits, axis)).quantize(xt, n_tokens, head_dim)
                c_ref, s_ref, z_ref = oracle.kv_cache_quantize(x, n_tokens, head_dim, bits, axis.value)
                tag = (n_tokens, head_dim, axis, bits)
                assert cache.n_groups() == len(s_ref)
                assert np.array_equal(_bits(cache.scales.cpu().numpy()), _bits(s_ref)), tag
                assert np.array_equal(_bits(cache.zero_points.cpu().numpy()), _bits(z_ref)), tag
                assert np.array_equal(cache.codes.cpu().numpy(), c_ref), tag
                deq = KvCacheQuantizer.dequantize(cache)
                d_ref = oracle.kv_cache_dequantize(c_ref, n_tokens, head_dim, axis.value, s_ref, z_ref)
                assert np.array_equal(_bits(deq.cpu().numpy()), _bits(d_ref)), tag
                deq16 = KvCacheQuantizer.dequantize(cache, torch.bfloat16)
                assert torch.equal(deq16.cpu(), torch.from_numpy(d_ref).to(torch.bfloat16)), tag


def test_kv_codes_on_rounding_ties(cuda, oracle):
    """Quotients on and next to half-integers, where the kernels leave their one-multiplication path for the exact
    division: rows whose scale is 1, 0.5 or an arbitrary value, with elements at (k + 0.5) * scale and a few ulp
    either side; NaN and infinities among the elements; a scale outside the range the reciprocal is trusted in."""
    from oxicuda_b200.kv_cache import KvAxis, KvCacheConfig, KvCacheQuantizer, KvQuantConfig, quantize_tokens
    rng = np.random.default_rng(25)
    d = 128
    rows = []
    for top in (255.0, 127.5, 3.1415927, 1e-3, 77.7, 1e35):
        scale = np.float32(top) / np.float32(255.0)
        ks = rng.integers(0, 255, d - 2).astype(np.float32)
        v = ((ks + np.float32(0.5)) * scale).astype(np.float32)
        for i in range(v.size):
            step = (i % 5) - 2                   # -2 .. +2 ulp
            for _ in range(abs(step)):
                v[i] = np.nextafter(v[i], np.float32(np.inf if step > 0 else -np.inf))
        rows.append(np.concatenate([[np.float32(0.0), np.float32(top)], v]).astype(np.float32))
    sym = rows[0] - np.float32(127.5)            # symmetric case: amax 127.5, elements k + 0.5 - 127.5 (ties of either sign)
    rows.append(sym.astype(np.float32))
    weird = rows[2].copy()
    weird[5], weird[6], weird[7] = np.nan, np.inf, -np.inf
    rows.append(weird)
    x = np.stack(rows).astype(np.float32)
    n = x.shape[0]
    xt = _t(x, cuda)
    for bits in (8, 4):
        for axis, arr, nt, hd in ((KvAxis.PerToken, x, n, d), (KvAxis.PerChannel, np.ascontiguousarray(x.T), d, n)):
            cache = KvCacheQuantizer(KvCacheConfig.new(bits, axis)).quantize(_t(arr, cuda), nt, hd)
            c_ref, s_ref, z_ref = oracle.kv_cache_quantize(arr, nt, hd, bits, axis.value)
            assert np.array_equal(_bits(cache.scales.cpu().numpy()), _bits(s_ref)), (bits, axis)
            assert np.array_equal(cache.codes.cpu().numpy(), c_ref), (bits, axis)
        for symmetric in (False, True):
            got = quantize_tokens(xt, KvQuantConfig.new(bits, symmetric))
            c_ref, s_ref, z_ref = oracle.kv_quantize_tokens(x, n, d, bits, symmetric)
            assert np.array_equal(_bits(got.scale.cpu().numpy()), _bits(s_ref)), (bits, symmetric)
            assert np.array_equal(got.codes.cpu().numpy().astype(np.int32).reshape(-1), c_ref), (bits, symmetric)


def test_kv_cache_reference_cases(cuda, kat):
    """The assertions of the reference's own unit tests (kv_cache.rs:333-459), run on the GPU path with host inputs."""
    from tests.golden.make_reference_kat import lcg
    from oxicuda_b200 import _lib
    from oxicuda_b200.kv_cache import KvAxis, KvCacheConfig, KvCacheQuantizer

    def rel_err(a, b):
        return float((a - b).abs().sum() / max(float(a.abs().sum()), 1e-8))

    k = kat["kv_cache"]
    for name in ("int8_per_token_round_trip", "int8_per_channel_round_trip", "int4_round_trip_coarser_but_bounded"):
        c = k[name]
        x = torch.tensor(lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"]), dtype=torch.float32)
        cache = KvCacheQuantizer(KvCacheConfig.new(c["bits"], KvAxis(c["axis"]))).quantize(x, c["n_tokens"], c["head_dim"])
        assert not cache.codes.is_cuda and cache.n_groups() == c["n_groups"]
        assert rel_err(x, KvCacheQuantizer.dequantize(cache)) < c["rel_err"], name
    c = k["per_channel_beats_per_token_on_key_outliers"]
    x = torch.tensor(lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"]), dtype=torch.float32).view(c["n_tokens"], c["head_dim"])
    x[:, c["outlier_col"]] = c["outlier_base"] + torch.arange(c["n_tokens"], dtype=torch.float32) * np.float32(c["outlier_step"])
    errs = []
    for cfg in (KvCacheConfig.keys_int8(), KvCacheConfig.values_int8()):
        cache = KvCacheQuantizer(cfg).quantize(x, c["n_tokens"], c["head_dim"])
        errs.append(rel_err(x.reshape(-1), KvCacheQuantizer.dequantize(cache)))
    assert errs[0] < errs[1]
    c = k["append_token_grows_cache"]
    q = KvCacheQuantizer(KvCacheConfig.values_int8())
    x = torch.tensor(lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"]), dtype=torch.float32)
    cache = q.quantize(x, c["n_tokens"], c["head_dim"])
    row = torch.tensor(lcg(c["head_dim"], c["row_seed"], c["amp"]), dtype=torch.float32)
    q.append_token(cache, row)
    assert cache.n_tokens == c["n_tokens"] + 1 and cache.scales.numel() == c["n_tokens"] + 1
    assert cache.codes.numel() == (c["n_tokens"] + 1) * c["head_dim"]
    assert rel_err(row, KvCacheQuantizer.dequantize(cache)[c["n_tokens"] * c["head_dim"]:]) < c["rel_err"]
    with pytest.raises(_lib.DimensionMismatch):
        q.append_token(cache, torch.ones(c["head_dim"] - 1))
    kq = KvCacheQuantizer(KvCacheConfig.keys_int8())
    with pytest.raises(_lib.InvalidConfig):
        kq.append_token(kq.quantize(x, c["n_tokens"], c["head_dim"]), row)
    c = k["packed_bytes_reflects_bit_width"]
    v = torch.tensor(lcg(c["n"], 9, 1.0), dtype=torch.float32)
    assert KvCacheQuantizer(KvCacheConfig.new(4, KvAxis.PerToken)).quantize(v, 4, 8).packed_bytes() == c["bits4_bytes"]
    assert KvCacheQuantizer(KvCacheConfig.new(8, KvAxis.PerToken)).quantize(v, 4, 8).packed_bytes() == c["bits8_bytes"]


def test_kv_cache_c_abi_errors(cuda):
    from oxicuda_b200 import _lib
    from oxicuda_b200._lib import default_handle, ptr
    h = default_handle()
    x = torch.ones(8, 8, device=cuda)
    codes = torch.empty(64, dtype=torch.uint8, device=cuda)
    s = torch.empty(8, device=cuda)
    z = torch.empty(8, device=cuda)
    with pytest.raises(_lib.EmptyInput):
        h.call("b2q_kv_cache_quantize_f32", ptr(x), 0, 8, 8, 0, ptr(codes), ptr(s), ptr(z))
    for bits in (1, 9, 16):
        with pytest.raises(_lib.InvalidBitWidth):
            h.call("b2q_kv_cache_quantize_f32", ptr(x), 8, 8, bits, 0, ptr(codes), ptr(s), ptr(z))
    with pytest.raises(_lib.InvalidConfig):
        h.call("b2q_kv_quantize_tokens_f32", ptr(x), 8, 8, 3, 0, ptr(codes), ptr(s), ptr(z))
    with pytest.raises(_lib.InvalidConfig):
        h.call("b2q_kv_quantize_tokens_f32", ptr(x), 0, 8, 8, 0, ptr(codes), ptr(s), ptr(z))
    with pytest.raises(_lib.InvalidArgument):
        h.call("b2q_kv_cache_quantize_f32", ptr(x), 8, 8, 8, 0, None, ptr(s), ptr(z))


@pytest.mark.parametrize("bf16", [False, True])
def test_kv_quantize_tokens_bit_exact(cuda, oracle, bf16):
    from oxicuda_b200.kv_cache import KvQuantConfig, quantize_tokens
    rng = np.random.default_rng(22)
    for n_tokens, d in ((1, 5), (3, 40), (64, 128), (1000, 96), (4096, 128), (17, 1026)):
        x = _kv_input(rng, n_tokens, d, bf16)
        x[0, :] = 0.0                                # all-zero vector: scale 1
        xt = _t(x, cuda).to(torch.bfloat16) if bf16 else _t(x, cuda)
        for symmetric in (False, True):
            for bits in (8, 4):
                cfg = KvQuantConfig.new(bits, symmetric)
                got = quantize_tokens(xt, cfg)
                c_ref, s_ref, z_ref = oracle.kv_quantize_tokens(x, n_tokens, d, bits, symmetric)
                tag = (n_tokens, d, symmetric, bits)
                lo, hi = cfg.q_range()
                assert int(got.codes.min()) >= lo and int(got.codes.max()) <= hi
                assert np.array_equal(_bits(got.scale.cpu().numpy()), _bits(s_ref)), tag
                assert np.array_equal(got.zero_point.cpu().numpy(), z_ref), tag
                assert np.array_equal(got.codes.cpu().numpy().astype(np.int32).reshape(-1), c_ref), tag
                d_ref = oracle.kv_dequantize_tokens(c_ref, n_tokens, d, s_ref, z_ref)
                assert np.array_equal(_bits(got.dequantize().cpu().numpy().reshape(-1)), _bits(d_ref)), tag


def test_kv_quant_reference_cases(cuda, kat):
    """The assertions of kv_quant.rs:195-290 through the single-vector mirror."""
    from oxicuda_b200 import _lib
    from oxicuda_b200.kv_cache import KvQuantConfig, quantization_mse, quantize_dequantize_token, quantize_token
    k = kat["kv_quant"]
    r = k["q_range_signed_and_unsigned"]
    assert list(KvQuantConfig.new(8, False).q_range()) == r["asym8"]
    assert list(KvQuantConfig.new(8, True).q_range()) == r["sym8"]
    assert list(KvQuantConfig.new(4, False).q_range()) == r["asym4"]
    with pytest.raises(_lib.InvalidConfig):
        KvQuantConfig.new(3, False)
    with pytest.raises(_lib.InvalidConfig):
        quantize_token([], KvQuantConfig.int8())
    c = k["asymmetric_endpoints_exact"]
    q = quantize_token(c["x"], KvQuantConfig.int8())
    rec = q.dequantize()
    assert q.zero_point == c["zero_point"] and abs(rec[0] - c["x"][0]) < c["tol"] and abs(rec[3] - c["x"][3]) < c["tol"]
    c = k["symmetric_zero_point_is_zero"]
    cfg = KvQuantConfig.new(8, True)
    assert quantize_token(c["x"], cfg).zero_point == 0.0 and quantization_mse(c["x"], cfg) < c["mse"]
    c = k["constant_vector_zero_error"]
    assert all(abs(v - c["x"][0]) < c["tol"] for v in quantize_dequantize_token(c["x"], KvQuantConfig.int8()))
    c = k["dequantize_matches_round_trip_helper"]
    assert quantize_token(c["x"], KvQuantConfig.int8()).dequantize() == quantize_dequantize_token(c["x"], KvQuantConfig.int8())
    c = k["mse_decreases_with_precision_on_smooth_signal"]
    x = [float(np.cos(np.float32(i) * np.float32(c["step"]))) for i in range(c["n"])]
    mse4, mse8 = quantization_mse(x, KvQuantConfig.new(4, False)), quantization_mse(x, KvQuantConfig.new(8, False))
    assert mse8 <= mse4 and mse8 < c["mse8"]
    x = [float(np.sin(np.float32(i) * np.float32(0.613)) * 2.7 + np.cos(np.float32(i) * np.float32(0.27)) * 1.3) for i in range(40)]
    assert 0.0 < quantization_mse(x, KvQuantConfig.new(8, False)) < quantization_mse(x, KvQuantConfig.new(4, False))


def _rms_reference(oracle, x, gamma, eps, residual, fmt_rne=True):
    """Oracle composition: RMSNorm in f32 (sequential sum), then the per-token FP8 rule of fp8_quantize_rows."""
    rows, cols = x.shape
    if residual is not None:
        summed = torch.from_numpy(residual + x).to(torch.bfloat16).to(torch.float32).numpy()   # the sum as it is stored
    else:
        summed = x
    y = oracle.rms_norm(summed, gamma, rows, cols, eps).reshape(rows, cols)
    return y, summed


@pytest.mark.parametrize("with_residual", [False, True])
def test_rms_norm_quantize_fp8(cuda, oracle, with_residual):
    from oxicuda_b200.kv_cache import rms_norm_quantize_fp8
    rng = np.random.default_rng(23)
    eps = 1e-5
    for rows, cols in ((1, 8), (3, 4096), (1, 8192), (64, 4096), (5, 16384), (300, 2048), (2, 32768), (7, 1000), (4, 40008), (1200, 1024)):
        x = torch.from_numpy((rng.standard_normal((rows, cols)) * 1.5).astype(np.float32)).to(torch.bfloat16)
        gamma = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)).to(torch.bfloat16)
        res = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).to(torch.bfloat16) if with_residual else None
        if rows > 2:
            x[2, :] = 0
            if res is not None:
                res[2, :] = 0
        y_ref, summed = _rms_reference(oracle, x.float().numpy(), gamma.float().numpy(), eps, None if res is None else res.float().numpy())
        res_dev = None if res is None else res.to(cuda)
        codes, scales, y = rms_norm_quantize_fp8(x.to(cuda), gamma.to(cuda), eps, residual=res_dev, want_y=True)
        torch.cuda.synchronize()
        tag = (rows, cols, with_residual)
        if res is not None:      # residual + x in f32, rounded once to bf16: bit-exact
            assert torch.equal(res_dev.cpu(), torch.from_numpy(summed).to(torch.bfloat16)), tag
        # y: f32 arithmetic whose only difference from the oracle is the order of the sum of squares (<= a few ulp of f32),
        # then one bf16 rounding: allow one bf16 ulp (2^-8 relative)
        y_got = y.float().cpu().numpy()
        assert np.all(np.abs(y_got - y_ref) <= np.abs(y_ref) * 2.0 ** -8 + 1e-30), tag
        # scales: absmax(y)/448 in f32; the oracle's sequential f32 sum of squares itself drifts by about
        # sqrt(cols) * 2^-24 relative, so the tolerance grows with the row length
        s_ref = np.where(np.abs(y_ref).max(axis=1) > 0, np.abs(y_ref).max(axis=1) / np.float32(448.0), 1.0)
        assert np.allclose(scales.cpu().numpy(), s_ref, rtol=1e-5 * max(1.0, cols / 4096), atol=0), tag
        # against an f64 statement of the same formula the kernel's tree sum is tight whatever the row length
        xs = summed.astype(np.float64)
        y64 = xs / np.sqrt((xs * xs).mean(axis=1, keepdims=True) + eps) * gamma.float().numpy().astype(np.float64)
        s64 = np.where(np.abs(y64).max(axis=1) > 0, np.abs(y64).max(axis=1) / 448.0, 1.0)
        assert np.allclose(scales.cpu().numpy(), s64, rtol=2e-6, atol=0), tag
        # codes: decode(code) * scale within half an E4M3 step (2^-4 relative) of y, plus the subnormal step near zero
        dec = oracle.fp8_decode(codes.cpu().numpy().reshape(-1), 0, 1).reshape(rows, cols) * scales.cpu().numpy()[:, None]
        tol = np.abs(y_ref) * 2.0 ** -4 + scales.cpu().numpy()[:, None] * 2.0 ** -10 + 1e-30
        assert np.all(np.abs(dec - y_ref) <= tol), tag
        # and bit-exact against the per-token quantizer applied to the kernel's own f32 y is not observable from outside;
        # the same call without y_out must give the same codes and scales
        codes2, scales2 = rms_norm_quantize_fp8(x.to(cuda), gamma.to(cuda), eps, residual=None if res is None else res.to(cuda))
        assert torch.equal(codes, codes2) and torch.equal(scales, scales2), tag


def test_rms_norm_quantize_feeds_fp8_gemm(cuda, oracle):
    """RMSNorm -> FP8 codes -> b2q_gemm_fp8 equals normalise, quantize per token, multiply in the oracle (<= 1e-2)."""
    from oxicuda_b200.blas import gemm_fp8
    from oxicuda_b200.kv_cache import rms_norm_quantize_fp8
    from oxicuda_b200.quant import Fp8Codec
    rng = np.random.default_rng(24)
    M, K, N = 16, 4096, 512
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16).to(cuda)
    gamma = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)).to(torch.bfloat16).to(cuda)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    wc, ws = Fp8Codec.e4m3("rne").quantize_rows(_t(w, cuda), N, K)
    codes, scales = rms_norm_quantize_fp8(x, gamma, 1e-6)
    out = gemm_fp8(codes, wc.view(N, K), scales, ws, out_dtype=torch.float32)
    ref = oracle.gemm_fp8(codes.cpu().numpy(), wc.cpu().numpy().reshape(N, K), scales.cpu().numpy(), ws.cpu().numpy(), 0, 1, want="f32")
    ref = np.asarray(ref).reshape(M, N)
    got = out.cpu().numpy()
    tau = 1e-3 * np.sqrt((ref ** 2).mean())
    assert (np.abs(got - ref) / np.maximum(np.abs(ref), tau)).max() <= 1e-2
