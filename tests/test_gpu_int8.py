"""GPU: the INT8 paths through the C ABI — bit-exact codes, scales, s32 accumulators and f32 outputs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _check_llm_int8(cuda, oracle, x, w, samples, rows, cols, threshold, row_wise=True):
    from oxicuda_b200.quant import LlmInt8Config, LlmInt8Quantizer
    q = LlmInt8Quantizer(LlmInt8Config(threshold, row_wise))
    got = q.matmul(_t(x, cuda), _t(w, cuda), samples, rows, cols, dump=True)
    ref = oracle.llm_int8_matmul(x, w, samples, rows, cols, threshold, row_wise)
    assert np.array_equal(got.s_w.cpu().numpy().view(np.uint32), ref["s_w"].view(np.uint32))
    assert np.array_equal(got.s_x.cpu().numpy().view(np.uint32), ref["s_x"].view(np.uint32))
    assert np.array_equal(got.w_q.cpu().numpy(), ref["w_q"])
    assert np.array_equal(got.x_q.cpu().numpy(), ref["x_q"])
    assert np.array_equal(got.acc.cpu().numpy(), ref["acc"])
    assert np.array_equal(got.output.cpu().numpy().view(np.uint32), ref["output"].view(np.uint32))
    assert got.outlier_columns == list(np.nonzero(ref["outlier_mask"])[0])
    return got, ref


def test_config1_w8a8_linear_bit_exact(cuda, oracle):
    """W 1024x1024 ~N(0,0.02), X 8x1024 ~N(0,1): int8 codes, scales, int32 accumulators and f32 output bit-exact."""
    rng = np.random.default_rng(0xB2000000)
    w = (rng.standard_normal((1024, 1024)) * 0.02).astype(np.float32)
    x = rng.standard_normal((8, 1024)).astype(np.float32)
    got, ref = _check_llm_int8(cuda, oracle, x, w, 8, 1024, 1024, 1e30)
    assert ref["n_outliers"] == 0 and got.outlier_fraction == 0.0
    assert np.abs(ref["acc"]).max() < 2**24            # the i64 -> f32 cast of the reference is exact here
    got6, ref6 = _check_llm_int8(cuda, oracle, x, w, 8, 1024, 1024, 6.0)
    assert ref6["n_outliers"] == 0
    assert np.array_equal(got6.output.cpu().numpy(), got.output.cpu().numpy())


def test_llm_int8_outliers_and_edge_cases(cuda, oracle, kat):
    rng = np.random.default_rng(21)
    # outlier columns, zero rows (scale 1.0), per-tensor activation scale, ragged sizes
    for samples, rows, cols in ((8, 64, 256), (1, 5, 16), (33, 17, 128), (64, 300, 1024)):
        w = (rng.standard_normal((rows, cols)) * 0.5).astype(np.float32)
        x = rng.standard_normal((samples, cols)).astype(np.float32)
        x[:, 7] += 40.0
        x[0, 3] = -9.0
        w[rows // 2] = 0.0
        if samples > 2:
            x[2] = 0.0
        for row_wise in (True, False):
            _, ref = _check_llm_int8(cuda, oracle, x, w, samples, rows, cols, 6.0, row_wise)
            assert ref["n_outliers"] >= 2
    c = kat["llm_int8"]["matmul_matches_fp32_when_no_outliers"]
    _check_llm_int8(cuda, oracle, np.array(c["x"], np.float32), np.array(c["w"], np.float32), c["samples"], c["rows"], c["cols"], 6.0)
    from oxicuda_b200.quant import LlmInt8Quantizer
    c = kat["llm_int8"]["outlier_fraction_reported"]
    out = LlmInt8Quantizer().matmul(torch.tensor(c["x"]), torch.tensor(c["w"]), c["samples"], c["rows"], c["cols"])
    assert abs(out.outlier_fraction - c["fraction"]) < 1e-6


def test_gemm_i8_exact_s32(cuda, oracle):
    from oxicuda_b200 import _lib
    from oxicuda_b200.blas import gemm_i8
    rng = np.random.default_rng(22)
    for M, N, K in ((8, 1024, 1024), (1, 64, 16), (33, 100, 260), (200, 136, 512), (64, 64, 4096), (256, 384, 1024), (130, 520, 144)):
        a = rng.integers(-128, 128, (M, K), dtype=np.int8)
        b = rng.integers(-128, 128, (N, K), dtype=np.int8)
        sa = rng.random(M).astype(np.float32) + 0.5
        sb = rng.random(N).astype(np.float32) + 0.5
        c32, cf = gemm_i8(_t(a, cuda), _t(b, cuda), _t(sa, cuda), _t(sb, cuda), want_s32=True, want_f32=True)
        ref = oracle.gemm_i8(a, b)
        assert np.array_equal(c32.cpu().numpy(), ref), (M, N, K)
        want_f = ref.astype(np.float32) * (sa[:, None] * sb[None, :])
        assert np.array_equal(cf.cpu().numpy().view(np.uint32), want_f.view(np.uint32)), (M, N, K)
    # saturating corners: all -128 x all -128 over K=4096 stays exact in s32
    a = np.full((128, 4096), -128, np.int8)
    c32, _ = gemm_i8(_t(a, cuda), _t(a, cuda))
    assert int(c32[0, 0]) == 128 * 128 * 4096 and bool((c32 == c32[0, 0]).all())
    with pytest.raises(_lib.InvalidDimension):                       # "K must be a multiple of 4", int_ops.rs:113-118
        gemm_i8(torch.zeros(4, 33, dtype=torch.int8, device=cuda), torch.zeros(4, 33, dtype=torch.int8, device=cuda))
    with pytest.raises(_lib.InvalidDimension):
        gemm_i8(torch.zeros(0, 32, dtype=torch.int8, device=cuda), torch.zeros(4, 32, dtype=torch.int8, device=cuda))
