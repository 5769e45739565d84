"""GPU: every quantize/dequantize kernel, through the C ABI, bit-exact against the CPU oracle and against
the reference's known-answer vectors."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _rng(seed):
    return np.random.default_rng(seed)


def test_minmax_calibrate_quantize_dequantize_bit_exact(cuda, oracle):
    from oxicuda_b200.quant import MinMaxQuantizer, QuantGranularity, QuantScheme
    rng = _rng(11)
    for rows, cols in ((1, 1), (1, 4099), (8, 1024), (1024, 1024), (3, 70001), (1, 1 << 20), (4096, 32)):
        x = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
        if x.size > 16:
            x[3] = 0.31
            x[-2] = -0.27
        for scheme in (QuantScheme.Symmetric, QuantScheme.Asymmetric):
            for bits in (8, 4):
                q = MinMaxQuantizer(bits, scheme, QuantGranularity.PerTensor())
                p = q.calibrate_2d(_t(x, cuda), rows, cols)
                s_ref, z_ref, st = oracle.minmax_calibrate(x, rows, cols, bits, scheme.value)
                assert st == 0
                assert np.array_equal(p.scales.cpu().numpy().view(np.uint32), s_ref.view(np.uint32)), (rows, cols, bits)
                assert np.array_equal(p.zero_points.cpu().numpy(), z_ref)
                codes = q.quantize_grouped(_t(x, cuda), p, cols)
                c_ref = oracle.minmax_quantize(x, rows, cols, s_ref, z_ref, bits, scheme.value)
                assert np.array_equal(codes.cpu().numpy(), c_ref)
                deq = q.dequantize_grouped(codes, p, cols)
                d_ref = oracle.minmax_dequantize(c_ref, rows, cols, s_ref, z_ref)
                assert np.array_equal(deq.cpu().numpy().view(np.uint32), d_ref.view(np.uint32))


def test_minmax_reference_pins_on_gpu(cuda, kat):
    from oxicuda_b200.quant import MinMaxQuantizer, QuantGranularity, QuantScheme
    k = kat["minmax"]
    c = k["symmetric_calibrate_scale"]
    p = MinMaxQuantizer.int8_symmetric().calibrate(torch.tensor(c["x"]))          # host in, host out
    assert abs(float(p.scales[0]) - c["scale"]) < c["eps"] and int(p.zero_points[0]) == 0
    c = k["asymmetric_calibrate_scale_zp"]
    p = MinMaxQuantizer(8, QuantScheme.Asymmetric, QuantGranularity.PerTensor()).calibrate(torch.tensor(c["x"]))
    assert abs(float(p.scales[0]) - c["scale"]) < c["eps"] and int(p.zero_points[0]) == 0
    c = k["per_group_calibrate"]
    assert MinMaxQuantizer.int4_per_group(c["group"]).calibrate(torch.tensor(c["x"])).scales.numel() == c["n_scales"]
    c = k["symmetric_round_trip_low_error"]
    t = torch.arange(c["n"], dtype=torch.float32) / (c["n"] - 1) * 2 - 1
    q = MinMaxQuantizer.int8_symmetric()
    p = q.calibrate(t)
    assert (q.dequantize(q.quantize(t, p), p) - t).abs().max() < c["max_err"]
    c = k["grouped_round_trip"]
    t = torch.arange(c["n"], dtype=torch.float32) * c["step"]
    q = MinMaxQuantizer.int4_per_group(c["group"])
    p = q.calibrate(t)
    assert (q.dequantize_grouped(q.quantize_grouped(t, p, c["group"]), p, c["group"]) - t).abs().max() < c["max_err"]
    from oxicuda_b200 import _lib
    with pytest.raises(_lib.GroupSizeMismatch):
        MinMaxQuantizer.int4_per_group(3).calibrate(torch.ones(10))


def test_invalid_scale_is_reported_from_the_device(cuda):
    from oxicuda_b200 import _lib
    from oxicuda_b200.quant import MinMaxQuantizer
    x = torch.full((64,), float("inf"), device=cuda)
    with pytest.raises(_lib.InvalidScale):
        MinMaxQuantizer.int8_symmetric().calibrate(x)


def test_fp8_codec_every_float_class(cuda, oracle, kat):
    from oxicuda_b200 import _lib
    from oxicuda_b200.quant import Fp8Codec
    rng = _rng(12)
    # dense sweep: every binade E4M3/E5M2 can see, both signs, plus random mantissas and exact ties
    mags = np.concatenate([np.ldexp(1.0 + rng.random(4000), rng.integers(-20, 18, 4000)),
                           np.ldexp(1.0 + np.arange(64) / 32.0, -3).repeat(2), [0.0, 448.0, 447.9, 464.0, 57344.0, 1e-10, 2**-9, 2**-10]])
    x = np.concatenate([mags, -mags]).astype(np.float32)
    for fmt, codec in ((0, Fp8Codec.e4m3), (1, Fp8Codec.e5m2)):
        for mode, name in ((0, "ref"), (1, "rne")):
            c = codec(name)
            got = c.encode(_t(x, cuda)).cpu().numpy()
            want, bad = oracle.fp8_encode(x, fmt, mode)
            assert bad == -1 and np.array_equal(got, want), (fmt, name, x[np.nonzero(got != want)[0][:5]])
            allc = np.arange(256, dtype=np.uint8)
            dec = c.decode(_t(allc, cuda)).cpu().numpy()
            assert np.array_equal(dec.view(np.uint32) & 0xFFBFFFFF, oracle.fp8_decode(allc, fmt, mode).view(np.uint32) & 0xFFBFFFFF)
    # reference pins through the CUDA path
    k = kat["fp8_codec"]
    assert list(Fp8Codec.e4m3().encode(torch.tensor(k["e4m3_zero"]["x"])).numpy()) == k["e4m3_zero"]["codes"]
    r = kat["fp8_rne"]["e4m3_encode_known_patterns"]
    assert list(Fp8Codec.e4m3("rne").encode(torch.tensor(r["x"])).numpy()) == r["codes"]
    for bad in (float("nan"), float("inf")):
        with pytest.raises(_lib.NonFiniteFp8):
            Fp8Codec.e4m3().encode(torch.tensor([1.0, bad, 2.0]))
    assert Fp8Codec.e4m3().encode(torch.empty(0)).numel() == 0
    data = torch.arange(256, dtype=torch.float32) / 128.0 - 1.0
    assert Fp8Codec.e4m3().quantization_mse(data) < k["mse_within_tolerance"]["mse"]


def test_fp8_quantize_rows_bit_exact(cuda, oracle):
    from oxicuda_b200.quant import Fp8Codec
    rng = _rng(13)
    for rows, cols, sigma in ((1, 1 << 18, 1.0), (64, 4096, 0.02), (7, 333, 1.0), (1, 1 << 22, 0.02), (3, 8, 0.0)):
        x = (rng.standard_normal(rows * cols) * sigma).astype(np.float32)
        for mode, name in ((0, "ref"), (1, "rne")):
            codes, scales = Fp8Codec.e4m3(name).quantize_rows(_t(x, cuda), rows, cols)
            c_ref, s_ref, bad = oracle.fp8_quantize_rows(x, rows, cols, 0, mode)
            assert bad == -1
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
            assert np.array_equal(codes.cpu().numpy(), c_ref)
    # bf16 activations take the same path
    xb = torch.randn(32, 4096, device=cuda, dtype=torch.bfloat16)
    codes, scales = Fp8Codec.e4m3("rne").quantize_rows(xb, 32, 4096)
    c_ref, s_ref, _ = oracle.fp8_quantize_rows(xb.float().cpu().numpy(), 32, 4096, 0, 1)
    assert np.array_equal(codes.cpu().numpy(), c_ref) and np.array_equal(scales.cpu().numpy(), s_ref)


@pytest.mark.parametrize("bf16", [False, True])
def test_fp8_quantize_rows_register_kernel_bit_exact(cuda, oracle, bf16):
    """Many rows of 256..16384 elements (a multiple of 8) take the kernel that keeps a row in registers: 1, 2 or 4 chunks
    per thread, rows that fill every thread and rows that do not, both roundings, a zero row and (f32) a NaN element."""
    from oxicuda_b200 import _lib
    from oxicuda_b200._lib import default_handle
    from oxicuda_b200.quant import Fp8Codec
    rng = _rng(14)
    for rows, cols in ((44, 256), (200, 1024), (64, 4096), (70, 8192), (3, 2048), (65, 1000), (130, 16384), (64, 4104)):
        x = torch.from_numpy((rng.standard_normal((rows, cols)) * rng.uniform(0.01, 3.0, (rows, 1))).astype(np.float32))
        x[1, :] = 0.0
        if bf16:
            x = x.to(torch.bfloat16)
        xf = x.float().numpy().reshape(-1)
        for mode, name in ((0, "ref"), (1, "rne")):
            codes, scales = Fp8Codec.e4m3(name).quantize_rows(x.to(cuda), rows, cols)
            c_ref, s_ref, bad = oracle.fp8_quantize_rows(xf, rows, cols, 0, mode)
            assert bad == -1
            assert np.array_equal(scales.cpu().numpy().view(np.uint32), s_ref.view(np.uint32)), (rows, cols, name)
            assert np.array_equal(codes.cpu().numpy(), c_ref), (rows, cols, name)
    if not bf16:
        x = torch.ones(64, 512)
        x[5, 17] = float("nan")
        Fp8Codec.e4m3("rne").quantize_rows(x.to(cuda), 64, 512)
        with pytest.raises(_lib.NonFiniteFp8):
            default_handle().check()


def test_fp4_block_quantize_bit_exact(cuda, oracle, kat):
    from oxicuda_b200.blas import Fp4Format, MicroScalingConfig, MicroScalingQuantizer, ScalingFormat
    rng = _rng(14)
    for n, sigma in ((32, 1.0), (4096 * 64, 0.02), (128 * 1001, 3.0)):
        x = (rng.standard_normal(n) * sigma).astype(np.float32)
        x[:32] = 0.0                                         # an all-zero block (scale 1.0)
        if n > 64:
            x[40] = np.float32(6.0) * np.abs(x[32:64]).max()  # exact multiples of the grid
        for block in (32, 64, 128):
            if n % block:
                continue
            for fmt in (Fp4Format.E2M1, Fp4Format.Int4):
                for sf, mode in ((ScalingFormat.Fp32, 0), (ScalingFormat.E8M0, 1)):
                    msq = MicroScalingQuantizer(MicroScalingConfig(block, sf))
                    packed, scales = msq.quantize_fp4(_t(x, cuda), fmt)
                    p_ref, s_ref = oracle.fp4_block_quantize(x, block, fmt.value, mode)
                    assert np.array_equal(scales.cpu().numpy().view(np.uint8), s_ref.view(np.uint8)), (n, block, fmt, sf)
                    assert np.array_equal(packed.cpu().numpy(), p_ref), (n, block, fmt, sf)
                    deq = msq.dequantize_fp4(packed, scales, fmt, n)
                    d_ref = oracle.fp4_block_dequantize(p_ref, s_ref, n, block, fmt.value)
                    assert np.array_equal(deq.cpu().numpy().view(np.uint32), d_ref.view(np.uint32))
    c = kat["fp4"]["fp4_e2m1_roundtrip_accuracy"]
    x = np.zeros(32, np.float32)
    x[:8] = c["x"]
    msq = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.Fp32))
    packed, scales = msq.quantize_fp4(torch.from_numpy(x), Fp4Format.E2M1)      # absmax 6 -> scale 1.0
    assert float(scales[0]) == 1.0
    assert np.array_equal(msq.dequantize_fp4(packed, scales, Fp4Format.E2M1, 32).numpy(), x)
    from oxicuda_b200 import _lib
    with pytest.raises(_lib.InvalidArgument):
        MicroScalingQuantizer(MicroScalingConfig(48)).quantize_fp4(torch.ones(96))


def test_nf4_bit_exact(cuda, oracle):
    from oxicuda_b200 import _lib
    from oxicuda_b200.quant import Nf4Quantizer
    rng = _rng(15)
    for block in (64, 32, 2, 128, 256, 24):          # 32..256: eight elements per lane; others: a warp per block
        x = rng.standard_normal(block * 513).astype(np.float32)
        x[:block] = 0.0
        q = Nf4Quantizer(block)
        packed, am = q.encode(_t(x, cuda))
        p_ref, a_ref = oracle.nf4_encode(x, block)
        assert np.array_equal(am.cpu().numpy().view(np.uint32), a_ref.view(np.uint32))
        assert np.array_equal(packed.cpu().numpy(), p_ref)
        dec = q.decode(packed, am)
        assert np.array_equal(dec.cpu().numpy().view(np.uint32), oracle.nf4_decode(p_ref, a_ref, block).view(np.uint32))
    with pytest.raises(_lib.GroupSizeMismatch):
        Nf4Quantizer(64).encode(torch.ones(100))
    with pytest.raises(_lib.DimensionMismatch):
        Nf4Quantizer(64).decode(torch.zeros(64, dtype=torch.uint8), torch.ones(3))


def test_int8_scalar_and_fake_quant_kernels(cuda, oracle):
    """int8_quant / int8_dequant / fake_quant_inplace on tie-free inputs, as the reference's GPU tests build them
    (crates/oxicuda-quant/src/gpu_tests.rs:121-131), plus explicit ties for the documented rounding of each."""
    from oxicuda_b200.quant import fake_quant_inplace, int8_dequant, int8_quant
    n = 4099
    scale = 0.05
    k = (np.arange(n) % 301 - 150).astype(np.float32)
    x = ((k + 0.3) * scale).astype(np.float32)
    q = int8_quant(_t(x, cuda), scale).cpu().numpy()
    assert np.array_equal(q, np.clip(np.rint(x / np.float32(scale)), -127, 127).astype(np.int8))
    assert list(int8_quant(torch.tensor([0.5, 1.5, 2.5, -0.5, 1000.0]), 1.0).numpy()) == [0, 2, 2, 0, 127]  # ties to even
    d = int8_dequant(_t(q, cuda), scale).cpu().numpy()
    assert np.array_equal(d, q.astype(np.float32) * np.float32(scale))
    xf = _t(x, cuda).clone()
    fake_quant_inplace(xf, scale, 0.0, -128.0, 127.0)
    assert np.array_equal(xf.cpu().numpy().view(np.uint32), oracle.fake_quant(x, scale, 0.0, -128.0, 127.0).view(np.uint32))
    t = torch.tensor([0.5, 1.5, 2.5, -0.5], device=cuda)
    fake_quant_inplace(t, 1.0, 0.0, -128.0, 127.0)
    assert t.tolist() == [1.0, 2.0, 3.0, -1.0]                                                      # half away from zero


def test_distfp8_bit_exact(cuda, oracle, kat):
    from oxicuda_b200 import _lib as L
    rng = _rng(16)
    h = L.default_handle()
    for n, block in ((4096, 4096), (4096, 64), (1 << 20, 1 << 20), (64 * 77, 64)):
        x = rng.standard_normal(n).astype(np.float32)
        x[:block if block < n else 0] = 0.0
        xd = _t(x, cuda)
        q = torch.empty(n, dtype=torch.uint8, device=cuda)
        am = torch.empty(n // block, dtype=torch.float32, device=cuda)
        h.call("b2q_distfp8_quantize_block_f32", L.ptr(xd), n, block, L.ptr(q), L.ptr(am))
        q_ref, a_ref = oracle.distfp8_quantize_block(x, block)
        assert np.array_equal(am.cpu().numpy(), a_ref) and np.array_equal(q.cpu().numpy(), q_ref)
        out = torch.empty(n, dtype=torch.float32, device=cuda)
        h.call("b2q_distfp8_dequantize_block_f32", L.ptr(q), n, block, L.ptr(am), L.ptr(out))
        assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle.distfp8_dequantize_block(q_ref, a_ref, block).view(np.uint32))
    for name in ("max_quantized_value_is_127", "negative_packs_as_twos_complement", "zero_quantizes_to_zero"):
        c = kat["distfp8"][name]
        xd = torch.tensor(c["x"], device=cuda)
        q = torch.empty(1, dtype=torch.uint8, device=cuda)
        am = torch.empty(1, dtype=torch.float32, device=cuda)
        h.call("b2q_distfp8_quantize_block_f32", L.ptr(xd), 1, 1, L.ptr(q), L.ptr(am))
        assert q.tolist() == c["q"]
