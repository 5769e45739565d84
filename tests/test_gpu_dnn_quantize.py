"""GPU: the oxicuda-dnn quantize surface through the C ABI — the reference's own GPU test cases
(crates/oxicuda-dnn/src/gpu_tests/quantize.rs) restated, and bit-exact parity with the CPU oracle on larger inputs."""
import numpy as np
import pytest
import torch

from tests.test_oracle_golden import DnnLcg

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _close(got, ref, rel, ab):
    return np.all(np.abs(got - ref) <= ab + rel * np.abs(ref))


def test_reference_gpu_test_cases(cuda, kat):
    from oxicuda_b200 import dnn_quantize as dq
    k = kat["dnn_quantize"]
    # int8_quantize_numeric
    c = k["int8_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    q, scale = dq.quantize_to_int8(_t(data, cuda))
    s = scale.cpu().numpy()[0]
    cpu_scale = max(np.float32(np.abs(data).max()) / np.float32(c["qmax"]), np.float32(c["scale_floor"]))
    assert _close(s, cpu_scale, c["scale_rel"], c["scale_abs"])
    expect = np.rint(np.clip(data / s, -127.0, 127.0)).astype(np.int8)          # np.rint rounds half to even
    assert np.array_equal(q.cpu().numpy(), expect)
    # int8_dequantize_numeric
    c = k["int8_dequantize_numeric"]
    lcg = DnnLcg(c["seed"])
    qv = np.array([(lcg.next_u32() % 255) - 127 for _ in range(c["n"])], np.int8)
    out = dq.dequantize_from_int8(_t(qv, cuda), torch.tensor([c["scale"]], device=cuda), c["n"])
    assert _close(out.cpu().numpy(), qv.astype(np.float32) * np.float32(c["scale"]), c["rel"], c["abs"])
    # fp8_quantize_numeric: the bytes against the hardware-independent E4M3 statement in torch (ties to even, saturating)
    c = k["fp8_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    codes, scale = dq.quantize_to_fp8(_t(data, cuda))
    s = scale.cpu().numpy()[0]
    cpu_scale = max(np.float32(np.abs(data).max()) / np.float32(c["qmax"]), np.float32(c["scale_floor"]))
    assert _close(s, cpu_scale, c["scale_rel"], c["scale_abs"])
    scaled = torch.from_numpy(np.clip(data / s, -448.0, 448.0).astype(np.float32))
    assert np.array_equal(codes.cpu().numpy(), scaled.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    # fp8_dequantize_numeric: every byte
    c = k["fp8_dequantize_numeric"]
    b = np.arange(256, dtype=np.uint8)
    out = dq.dequantize_from_fp8(_t(b, cuda), torch.tensor([c["scale"]], device=cuda), 256).cpu().numpy()
    ref = torch.from_numpy(b).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    ref[0x7F], ref[0xFF] = 480.0, -480.0              # the reference's decoder has no NaN slot (quantize.rs:112-125)
    assert _close(out, ref * np.float32(c["scale"]), c["rel"], c["abs"])
    # block_quantize_numeric
    c = k["block_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    out, scales = dq.quantize_block_scaled(_t(data, cuda), c["block"])
    sc = scales.cpu().numpy()
    cpu_scales = np.maximum(np.abs(data).reshape(-1, c["block"]).max(axis=1) / np.float32(c["qmax"]), np.float32(c["scale_floor"]))
    assert _close(sc, cpu_scales, c["scale_rel"], c["scale_abs"])
    expect = np.clip(np.rint(np.clip(data / np.repeat(sc, c["block"]), -6.0, 6.0)).astype(np.int32) + 6, 0, 255).astype(np.uint8)
    assert np.array_equal(out.cpu().numpy(), expect)


def test_bit_exact_against_oracle(cuda, oracle):
    from oxicuda_b200 import dnn_quantize as dq
    rng = np.random.default_rng(31)
    for n in (1, 5, 257, 4096, 70001, 1 << 20):
        x = (rng.standard_normal(n) * 3.0).astype(np.float32)
        if n > 16:
            x[3], x[7], x[11] = 0.0, np.float32(1e-7), -x[5]
        xt = _t(x, cuda)
        codes, s = dq.quantize_to_fp8(xt)
        c_ref, s_ref = oracle.dnn_quantize_to_fp8(x)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32)) and np.array_equal(codes.cpu().numpy(), c_ref), n
        d_ref = oracle.dnn_dequantize_from_fp8(c_ref, s_ref[0])
        assert np.array_equal(dq.dequantize_from_fp8(codes, s).cpu().numpy().view(np.uint32), d_ref.view(np.uint32)), n
        q, s = dq.quantize_to_int8(xt)
        q_ref, s_ref = oracle.dnn_quantize_to_int8(x)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32)) and np.array_equal(q.cpu().numpy(), q_ref), n
        d_ref = oracle.dnn_dequantize_from_int8(q_ref, s_ref[0])
        assert np.array_equal(dq.dequantize_from_int8(q, s).cpu().numpy().view(np.uint32), d_ref.view(np.uint32)), n
        for block in (16, 32, 128):
            out, sc = dq.quantize_block_scaled(xt, block)
            o_ref, sc_ref = oracle.dnn_quantize_block_scaled(x, block)
            assert np.array_equal(sc.cpu().numpy().view(np.uint32), sc_ref.view(np.uint32)) and np.array_equal(out.cpu().numpy(), o_ref), (n, block)
        for block in (3, 64, 100, 128):
            bq = dq.BlockQuantizedInt8.quantize(xt, block)
            q_ref, sc_ref = oracle.block_int8_quantize(x, block)
            assert np.array_equal(bq.scales.cpu().numpy().view(np.uint32), sc_ref.view(np.uint32)), (n, block)
            assert np.array_equal(bq.data.cpu().numpy(), q_ref), (n, block)
            d_ref = oracle.block_int8_dequantize(q_ref, sc_ref, block)
            assert np.array_equal(bq.dequantize().cpu().numpy().view(np.uint32), d_ref.view(np.uint32)), (n, block)
        sc = dq.Fp4BlockQuantizer.new(32).compute_scales(xt)
        assert np.array_equal(sc.cpu().numpy().view(np.uint32), oracle.block_absmax_scale(x, 32, 6.0).view(np.uint32)), n
    # an all-zero tensor: scale 1e-12 (the floor), codes zero
    z = torch.zeros(1000, device=cuda)
    codes, s = dq.quantize_to_fp8(z)
    assert s.item() == np.float32(1e-12) and int(codes.max()) == 0
    # NaN elements follow the CPU statements (NaN -> 0x7E | sign for FP8, 0 for INT8).  Infinite elements make the scale
    # infinite and inf / inf a freshly generated NaN, whose sign bit differs between x86 and the GPU (as does the sign of
    # a NaN that passes through a division): only a positive NaN is compared.
    w = np.array([1.0, np.nan, -2.0, 7.5, 0.5, np.nan, 3.0, 0.25], np.float32)
    for fn_gpu, fn_ref in ((dq.quantize_to_fp8, oracle.dnn_quantize_to_fp8), (dq.quantize_to_int8, oracle.dnn_quantize_to_int8)):
        got, s = fn_gpu(_t(w, cuda))
        ref, s_ref = fn_ref(w)
        assert np.array_equal(got.cpu().numpy(), ref) and np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))


def test_block_int8_and_fp4_block_reference_cases(cuda, kat):
    """The CPU unit tests of BlockQuantizedInt8 (int8_quantize.rs:525-722) and Fp4BlockQuantizer (block_scale.rs:497-622)
    through the mirror, with host tensors in and out."""
    from oxicuda_b200 import _lib
    from oxicuda_b200.dnn_quantize import BlockQuantizedInt8, Fp4BlockQuantizer, quantize_block_scaled
    k = kat["dnn_quantize"]
    c = k["block_int8_round_trip"]
    x = (torch.arange(c["n"], dtype=torch.float32) - c["offset"]) / c["div"]
    bq = BlockQuantizedInt8.quantize(x, c["block"])
    deq = bq.dequantize()
    assert not deq.is_cuda and deq.numel() == c["n"] and float((deq - x).abs().max()) < c["tol"]
    assert bq.compression_ratio() > 3.0
    c = k["block_int8_non_multiple_len"]
    bq = BlockQuantizedInt8.quantize(torch.arange(c["n"], dtype=torch.float32), c["block"])
    assert bq.dequantize().numel() == c["n"] and bq.num_blocks() == c["num_blocks"]
    c = k["block_int8_max_value_saturation"]
    deq = BlockQuantizedInt8.quantize(torch.tensor(c["x"]), c["block"]).dequantize()
    assert deq[0] > 0 and deq[1] < 0 and deq[2] == 0
    c = k["block_int8_gptq_dequant_precision"]
    deq = BlockQuantizedInt8(torch.tensor(c["data"], dtype=torch.int8), torch.tensor([c["scale"]]), 3, 3).dequantize()
    assert float((deq - torch.tensor(c["expected"])).abs().max()) < c["tol"]
    c = k["block_int8_block_size_100_round_trip"]
    x = (torch.arange(c["n"], dtype=torch.float32) - c["offset"]) / c["div"]
    bq = BlockQuantizedInt8.quantize(x, c["block"])
    assert bq.num_blocks() == c["num_blocks"]
    assert float((bq.dequantize() - x).abs().max()) <= float(bq.scales.max()) * 0.5 + 1e-5
    c = k["block_int8_zero_input"]
    assert float(BlockQuantizedInt8.quantize(torch.zeros(c["n"]), c["block"]).dequantize().abs().max()) == 0.0
    c = k["fp4_block_quantizer"]
    for bad in c["bad"]:
        with pytest.raises(_lib.InvalidArgument):
            Fp4BlockQuantizer.new(bad)
    q = Fp4BlockQuantizer.new(c["ok"][0])
    assert q.compute_scale([0.0] * 32) == c["zeros_scale"] and abs(q.compute_scale([6.0] * 32) - c["six_scale"]) < 1e-6
    assert abs(q.compute_scale([12.0] * 32) - c["twelve_scale"]) < 1e-6 and Fp4BlockQuantizer.MAX_VALUE == c["max_value"]
    assert abs(q.compute_scale([-6.0, 3.0, 1.5] + [0.0] * 29) - 1.0) < 1e-6
    for n, want in c["num_scales"]:
        assert q.num_scales(n) == want
    for bad in k["block_size_validation"]["bad"]:
        with pytest.raises(_lib.InvalidArgument):
            quantize_block_scaled(torch.ones(64), bad)
    for ok in k["block_size_validation"]["ok"]:
        quantize_block_scaled(torch.ones(256), ok)
