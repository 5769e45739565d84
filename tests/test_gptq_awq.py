"""GPTQ / AWQ weight-only quantization (crates/oxicuda-dnn/src/quantize/gptq_awq.rs).

CPU: the host mirror against the reference's own unit tests (gptq_awq.rs:1203-1520), the oracle's restatement of the
five generated kernels against the closed forms the reference's GPU tests compare with
(crates/oxicuda-dnn/src/gpu_tests/quantize.rs:783-903) and against the packing rule written out in numpy.
GPU: every kernel through the C ABI bit-exact against the oracle (the scale search within 4 ulp: rsqrt.approx)."""
import numpy as np
import pytest
import torch


def _plan(rows, cols, group, bits=4, symmetric=True):
    from oxicuda_b200.gptq_awq import GptqConfig, WeightQuantMethod, WeightQuantPlan
    return WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig(bits=bits, group_size=group, block_size=group, symmetric=symmetric)), rows, cols)


def _awq_plan(rows, cols, group, bits=4, zero_point=True):
    from oxicuda_b200.gptq_awq import AwqConfig, WeightQuantMethod, WeightQuantPlan
    return WeightQuantPlan.new(WeightQuantMethod.Awq(AwqConfig(bits=bits, group_size=group, zero_point=zero_point)), rows, cols)


def pack_flat(codes, bits):
    """Element e of the flat matrix in word e / epu at bits [(e % epu) * bits, +bits) (gptq_awq.rs:471-489)."""
    epu = 32 // bits
    words = np.zeros(-(-codes.size // epu), np.uint64)
    for e, q in enumerate(codes.reshape(-1).astype(np.uint64)):
        words[e // epu] |= q << np.uint64((e % epu) * bits)
    return words.astype(np.uint32)


class Lcg:
    """The generator of the reference's GPU tests (crates/oxicuda-dnn/src/gpu_tests/mod.rs:169-194)."""

    def __init__(self, seed):
        self.state = seed

    def next_u32(self):
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        return self.state >> 32

    def range_f32(self, lo, hi):
        return np.float32(lo + (hi - lo) * (self.next_u32() / 4294967296.0))


def reference_gpu_test_inputs(seed, scale_hi, with_x):
    """The operands of gptq_dequantize_numeric (seed 0xABCD_1234, scales in [0.02, 0.4)) and fused_dequant_gemv_numeric
    (seed 0x55AA_9933, scales in [0.02, 0.3), x in [-2, 2)): 3 x 64, groups of 32, drawn in the reference's order
    (gpu_tests/quantize.rs:789-799, :846-857)."""
    rows, cols, group = 3, 64, 32
    lcg = Lcg(seed)
    nib = np.array([lcg.next_u32() % 16 for _ in range(rows * cols)], np.uint32)
    scales = np.array([lcg.range_f32(0.02, scale_hi) for _ in range(rows * (cols // group))], np.float32)
    x = np.array([lcg.range_f32(-2.0, 2.0) for _ in range(cols)], np.float32) if with_x else None
    return rows, cols, group, nib, scales, x


# ---------------------------------------------------------------------------
# host mirror: the reference's unit tests
# ---------------------------------------------------------------------------
def test_config_validation():
    """gptq_awq.rs:1207-1277"""
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.gptq_awq import AwqConfig, GptqConfig
    GptqConfig(bits=4, group_size=128, block_size=128, damp_percent=0.01, symmetric=True, act_order=False, true_sequential=True).validate()
    with pytest.raises(L.InvalidArgument, match="bits must be 2, 3, 4, or 8"):
        GptqConfig(bits=5).validate()
    with pytest.raises(L.InvalidArgument):
        GptqConfig(group_size=0).validate()
    AwqConfig(bits=4, group_size=128, zero_point=True, search_alpha_min=0.0, search_alpha_max=1.0, search_steps=20).validate()
    with pytest.raises(L.InvalidArgument):
        AwqConfig(bits=3).validate()
    with pytest.raises(L.InvalidArgument, match="alpha_min"):
        AwqConfig(search_alpha_min=1.0, search_alpha_max=0.0).validate()


def test_quantized_weight_info_and_plan_numbers():
    """gptq_awq.rs:1280-1331, :1455-1520"""
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.gptq_awq import AwqConfig, GptqConfig, QuantMethodTag, WeightQuantMethod, WeightQuantPlan
    info = WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig(bits=4, group_size=128, symmetric=True)), 256, 1024).quantized_weight_info()
    assert (info.bits, info.rows, info.cols, info.packed_weight_elements, info.scale_elements) == (4, 256, 1024, 32768, 2048)
    assert not info.has_zero_point and info.zero_point_elements == 0 and info.method == QuantMethodTag.Gptq
    info = WeightQuantPlan.new(WeightQuantMethod.Awq(AwqConfig(bits=8, group_size=128, zero_point=True)), 128, 512).quantized_weight_info()
    assert (info.bits, info.packed_weight_elements, info.scale_elements, info.zero_point_elements) == (8, 16384, 512, 512)
    assert info.has_zero_point and info.method == QuantMethodTag.Awq
    plan = WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig(block_size=128, act_order=True)), 256, 1024)
    assert plan.workspace_bytes() == 1024 * 4 + 1024 * 4 + 256 * 128 * 4
    assert WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig(block_size=128)), 64, 128).shared_memory_bytes() == 128 * 4
    assert WeightQuantPlan.new(WeightQuantMethod.Awq(AwqConfig(group_size=64)), 64, 128).shared_memory_bytes() == 64 * 4
    assert WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig()), 512, 1024).launch_params() == (2, 256)
    with pytest.raises(L.InvalidArgument, match="divisible"):
        WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig(group_size=100)), 64, 256)
    with pytest.raises(L.InvalidDimension):
        WeightQuantPlan.new(WeightQuantMethod.Gptq(GptqConfig()), 0, 256)
    with pytest.raises(L.InvalidArgument, match="called on AWQ plan"):
        WeightQuantPlan.new(WeightQuantMethod.Awq(AwqConfig()), 64, 128).gptq_quantize(torch.zeros(64 * 128), torch.zeros(128))
    # the C ABI's word count is quantized_weight_info's
    lib = L.lib()
    for rows, cols, bits in [(256, 1024, 4), (128, 512, 8), (3, 7, 3), (5, 33, 2)]:
        assert lib.b2q_wq_packed_words(rows, cols, bits) == -(-rows * cols // (32 // bits))
    assert lib.b2q_wq_packed_words(4, 4, 5) == -1


def test_gptq_state_and_awq_channel_scales():
    """gptq_awq.rs:1334-1409"""
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.gptq_awq import AwqChannelScales, GptqConfig, GptqState
    st = GptqState.new(256, 1024, GptqConfig())
    assert (st.rows, st.cols, st.columns_processed, st.quantization_error) == (256, 1024, 0, 0.0) and not st.is_complete()
    st = GptqState.new(128, 512, GptqConfig(group_size=64))
    assert st.num_groups() == 8 and st.num_column_blocks() == 8
    st = GptqState.new(64, 256, GptqConfig())
    st.columns_processed = 256
    assert st.is_complete()
    for bits, expected in [(2, 16), (3, 10), (4, 8), (8, 4)]:
        assert GptqState.new(64, 128, GptqConfig(bits=bits)).elements_per_packed_word() == expected
    sc = AwqChannelScales.new(128)
    assert sc.num_channels == 128 and len(sc.scales) == 128 and sc.scales[0] == 1.0
    sc = AwqChannelScales.new(4)
    sc.set_scale(2, 3.19)
    assert abs(sc.scales[2] - 3.19) < 1e-6
    with pytest.raises(L.InvalidArgument):
        sc.set_scale(4, 1.0)
    sc = AwqChannelScales.new(3)
    sc.scales = [4.0, 9.0, 16.0]
    sc.apply_alpha(0.5)
    assert sc.best_alpha == 0.5 and all(abs(a - b) < 1e-5 for a, b in zip(sc.scales, (2.0, 3.0, 4.0)))


# ---------------------------------------------------------------------------
# the oracle against closed forms
# ---------------------------------------------------------------------------
def test_oracle_dequantize_and_gemv_closed_forms(oracle):
    """The shapes and closed forms of gpu_tests/quantize.rs:783-903 (3 x 64, groups of 32, 4-bit), and every bit width."""
    rng = np.random.default_rng(5)
    rows, cols, group = 3, 64, 32
    gpr = cols // group
    nib = rng.integers(0, 16, rows * cols).astype(np.uint32)
    packed = pack_flat(nib, 4)
    scales = rng.uniform(0.02, 0.4, rows * gpr).astype(np.float32)
    x = rng.uniform(-2, 2, cols).astype(np.float32)
    deq = oracle.wq_dequantize(packed, scales, None, rows, cols, group, 4)
    expect = nib.astype(np.float32) * np.repeat(scales.reshape(rows, gpr), group, axis=1).reshape(-1)
    assert np.array_equal(deq, expect)
    y = oracle.fused_dequant_gemv(packed, scales, None, x, rows, cols, group, 4)
    ref = np.zeros(rows, np.float32)
    for r in range(rows):
        acc = np.float32(0)
        for c in range(cols):
            dq = np.float32(nib[r * cols + c]) * scales[r * gpr + c // group]
            acc = np.float32(np.float64(dq) * np.float64(x[c]) + np.float64(acc))        # fma: one rounding (the product is exact in f64)
        ref[r] = acc
    assert np.array_equal(y, ref)
    for bits, cols in [(2, 64), (3, 640), (8, 64)]:
        group = 32 if bits != 3 else 128
        q = rng.integers(0, 1 << bits, rows * cols).astype(np.uint32)
        s = rng.uniform(0.02, 0.4, rows * (cols // group)).astype(np.float32)
        z = rng.uniform(0, (1 << bits) - 1, rows * (cols // group)).astype(np.float32)
        sx = np.repeat(s.reshape(rows, -1), group, axis=1).reshape(-1)
        zx = np.repeat(z.reshape(rows, -1), group, axis=1).reshape(-1)
        assert np.array_equal(oracle.wq_dequantize(pack_flat(q, bits), s, None, rows, cols, group, bits), q.astype(np.float32) * sx)
        assert np.array_equal(oracle.wq_dequantize(pack_flat(q, bits), s, z, rows, cols, group, bits), (q.astype(np.float32) - zx) * sx)


def test_oracle_on_the_reference_gpu_test_inputs(oracle):
    """gptq_dequantize_numeric and fused_dequant_gemv_numeric (gpu_tests/quantize.rs:783-903) on their own operands: the
    oracle equals the reference tests' CPU expressions exactly (their bounds are 1e-5 and 1e-4 relative)."""
    rows, cols, group, nib, scales, _ = reference_gpu_test_inputs(0xABCD_1234, 0.4, False)
    gpr = cols // group
    cpu = np.array([np.float32(nib[e]) * scales[(e // cols) * gpr + (e % cols) // group] for e in range(rows * cols)], np.float32)
    assert np.array_equal(oracle.wq_dequantize(pack_flat(nib, 4), scales, None, rows, cols, group, 4), cpu)
    rows, cols, group, nib, scales, x = reference_gpu_test_inputs(0x55AA_9933, 0.3, True)
    cpu = np.zeros(rows, np.float32)
    for r in range(rows):
        acc = np.float32(0)
        for c in range(cols):
            dq = np.float32(nib[r * cols + c]) * scales[r * gpr + c // group]
            acc = np.float32(np.float64(dq) * np.float64(x[c]) + np.float64(acc))        # f32::mul_add
        cpu[r] = acc
    assert np.array_equal(oracle.fused_dequant_gemv(pack_flat(nib, 4), scales, None, x, rows, cols, group, 4), cpu)


def test_oracle_quantizers_closed_forms(oracle):
    """dnn_gptq_quantize_f32 / dnn_awq_* written out in numpy (round-half-even, the clamps in the kernel's order)."""
    rng = np.random.default_rng(6)
    rows, cols, group = 4, 32, 32
    w = rng.uniform(-1, 1, rows * cols).astype(np.float32)
    hd = rng.uniform(0.1, 2.0, cols).astype(np.float32)
    hd[3] = 0.0                                                          # below MIN_DAMP: the divisor becomes 1e-6
    for bits, sym in [(4, True), (4, False), (8, True), (2, False), (3, True)]:
        packed, scales = oracle.gptq_quantize(w, hd, rows, cols, group, bits, sym)
        safe = np.maximum(hd, np.float32(1e-6))
        r = np.rint(w.reshape(rows, cols) / safe).astype(np.float32)
        qmax = np.float32((1 << bits) - 1)
        if sym:
            r = np.maximum(r + np.float32(1 << (bits - 1)), np.float32(0))
        q = np.maximum(np.minimum(r, qmax), np.float32(0)).astype(np.uint32)
        assert np.array_equal(packed, pack_flat(q, bits)), (bits, sym)
        assert np.array_equal(scales, np.tile(safe[group - 1::group] / qmax, rows))
    cs = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    gs = rng.uniform(0.05, 0.5, rows).astype(np.float32)
    for bits in (4, 8):
        packed, zeros = oracle.awq_quantize(w, cs, gs, rows, cols, group, bits, True)
        r = np.rint((w.reshape(rows, cols) * cs) / np.maximum(gs, np.float32(1e-12))[:, None]).astype(np.float32)
        q = np.minimum(np.maximum(r, np.float32(0)), np.float32((1 << bits) - 1)).astype(np.uint32)
        assert np.array_equal(packed, pack_flat(q, bits)) and not zeros.any()
    act = np.concatenate([rng.uniform(0.01, 4.0, 40), [0.0, -2.25, 1e-9]]).astype(np.float32)
    sc = oracle.awq_scale_search(act)
    assert np.allclose(sc, np.sqrt(np.maximum(np.abs(act), np.float32(1e-7))), rtol=3e-7, atol=0)


# ---------------------------------------------------------------------------
# GPU parity
# ---------------------------------------------------------------------------
def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,sym,rows,cols,group", [(4, True, 4, 32, 32), (4, False, 4, 32, 32), (8, True, 37, 256, 64), (2, False, 5, 96, 32),
                                                      (3, True, 7, 128, 64), (3, False, 3, 640, 128), (4, True, 512, 4096, 128)])
def test_gptq_quantize_and_dequantize_bit_exact(cuda, oracle, bits, sym, rows, cols, group):
    rng = np.random.default_rng(bits * 100 + rows)
    w = rng.uniform(-1, 1, rows * cols).astype(np.float32) * rng.choice([0.2, 1.0, 8.0], rows * cols).astype(np.float32)
    hd = rng.uniform(0.05, 2.0, cols).astype(np.float32)
    hd[cols // 2] = 0.0
    hd[group - 1] = 1e-9
    plan = _plan(rows, cols, group, bits, sym)
    packed, scales = plan.gptq_quantize(_t(w, cuda), _t(hd, cuda))
    ref_packed, ref_scales = oracle.gptq_quantize(w, hd, rows, cols, group, bits, sym)
    assert np.array_equal(_u32(packed), ref_packed)
    assert np.array_equal(scales.cpu().numpy(), ref_scales)
    zeros = None if sym else rng.uniform(0, (1 << bits) - 1, rows * (cols // group)).astype(np.float32)
    deq = plan.gptq_dequantize(packed, scales, None if sym else _t(zeros, cuda))
    ref = oracle.wq_dequantize(ref_packed, ref_scales, zeros, rows, cols, group, bits)
    assert np.array_equal(deq.cpu().numpy().reshape(-1), ref)
    deq16 = plan.gptq_dequantize(packed, scales, None if sym else _t(zeros, cuda), out_dtype=torch.bfloat16)
    assert torch.equal(deq16.cpu().reshape(-1), torch.from_numpy(ref).to(torch.bfloat16))


@pytest.mark.gpu
def test_reference_gpu_test_cases(cuda, oracle):
    """gptq_dequantize_numeric and fused_dequant_gemv_numeric on the reference tests' own operands
    (gpu_tests/quantize.rs:783-903; bounds there 1e-5 and 1e-4 relative): equal to the oracle bit for bit."""
    rows, cols, group, nib, scales, _ = reference_gpu_test_inputs(0xABCD_1234, 0.4, False)
    packed = pack_flat(nib, 4)
    out = _plan(rows, cols, group).gptq_dequantize(_t(packed.view(np.int32), cuda), _t(scales, cuda))
    assert np.array_equal(out.cpu().numpy().reshape(-1), oracle.wq_dequantize(packed, scales, None, rows, cols, group, 4))
    rows, cols, group, nib, scales, x = reference_gpu_test_inputs(0x55AA_9933, 0.3, True)
    packed = pack_flat(nib, 4)
    y = _plan(rows, cols, group).fused_dequant_gemv(_t(packed.view(np.int32), cuda), _t(scales, cuda), _t(x, cuda))
    assert np.array_equal(y.cpu().numpy(), oracle.fused_dequant_gemv(packed, scales, None, x, rows, cols, group, 4))


@pytest.mark.gpu
def test_awq_kernels(cuda, oracle):
    """gpu_tests/quantize.rs:956-1085 launch the two AWQ kernels without checking values (4 x 32, groups of 32); here the
    quantizer is bit-exact against the restated kernel and the scale search within 4 ulp of sqrt."""
    rng = np.random.default_rng(77)
    for rows, cols, group, bits, zp in [(4, 32, 32, 4, True), (33, 512, 128, 8, False), (256, 2048, 64, 4, True)]:
        w = rng.uniform(-1, 1, rows * cols).astype(np.float32)
        cs = rng.uniform(0.5, 1.5, cols).astype(np.float32)
        gs = rng.uniform(0.05, 0.5, rows * (cols // group)).astype(np.float32)
        gs[0] = 0.0
        plan = _awq_plan(rows, cols, group, bits, zp)
        packed, zeros = plan.awq_quantize(_t(w, cuda), _t(cs, cuda), _t(gs, cuda))
        ref_packed, _ = oracle.awq_quantize(w, cs, gs, rows, cols, group, bits, zp)
        assert np.array_equal(_u32(packed), ref_packed)
        assert (zeros is None) == (not zp) and (zeros is None or not zeros.cpu().numpy().any())
        deq = plan.dequantize(packed, _t(gs, cuda), zeros)
        assert np.array_equal(deq.cpu().numpy().reshape(-1), oracle.wq_dequantize(ref_packed, gs, None, rows, cols, group, bits))
    act = np.concatenate([rng.uniform(0.01, 4.0, 1000), [0.0, -2.25, 1e-9, 3e38]]).astype(np.float32)
    got = _awq_plan(4, 32, 32).awq_scale_search(_t(act, cuda)).cpu().numpy()
    ref = oracle.awq_scale_search(act)
    assert np.all(np.isfinite(got)) and np.all(got >= 0)
    assert np.all(np.abs(got - ref) <= 4 * np.spacing(ref))


@pytest.mark.gpu
@pytest.mark.parametrize("bits,rows,cols,group", [(4, 3, 64, 32), (4, 300, 4096, 128), (8, 130, 1024, 64), (2, 129, 2048, 32), (3, 5, 640, 128),
                                                  (3, 200, 1280, 64), (4, 1000, 8192, 128), (4, 64, 96, 32),
                                                  (4, 7, 40, 8), (8, 9, 36, 12), (2, 3, 48, 16)])      # rows of 5, 9, 3 words: 4-byte copies
def test_fused_dequant_gemv_reference_order_bit_exact(cuda, oracle, bits, rows, cols, group):
    """gpu_tests/quantize.rs:840-903 (3 x 64, groups of 32; bound 1e-4) and larger, ragged shapes: the sum runs in the
    reference's order, so the result equals the restated kernel's bit for bit; with zero points likewise."""
    rng = np.random.default_rng(bits * 1000 + rows)
    q = rng.integers(0, 1 << bits, rows * cols).astype(np.uint32)
    packed = pack_flat(q, bits) if rows * cols < 200000 else None
    if packed is None:                                           # vectorised packing for the large cases (epu divides cols)
        epu = 32 // bits
        packed = (q.reshape(-1, epu).astype(np.uint64) << (np.arange(epu, dtype=np.uint64) * np.uint64(bits))).sum(axis=1).astype(np.uint32)
    scales = rng.uniform(0.02, 0.3, rows * (cols // group)).astype(np.float32)
    zeros = rng.uniform(0, (1 << bits) - 1, rows * (cols // group)).astype(np.float32)
    x = rng.uniform(-2, 2, cols).astype(np.float32)
    plan = _plan(rows, cols, group, bits)
    dp, ds, dz, dx = _t(packed.view(np.int32), cuda), _t(scales, cuda), _t(zeros, cuda), _t(x, cuda)
    y = plan.fused_dequant_gemv(dp, ds, dx).cpu().numpy()
    ref = oracle.fused_dequant_gemv(packed, scales, None, x, rows, cols, group, bits)
    assert np.array_equal(y, ref)
    yz = plan.fused_dequant_gemv(dp, ds, dx, zeros=dz).cpu().numpy()
    refz = oracle.fused_dequant_gemv(packed, scales, zeros, x, rows, cols, group, bits)
    assert np.array_equal(yz, refz)
    # split columns: another association of the same sum, deterministic
    for split in (0, 2, 8):
        ys = plan.fused_dequant_gemv(dp, ds, dx, split_k=split).cpu().numpy()
        assert np.allclose(ys, ref, rtol=1e-4, atol=1e-4 * float(np.abs(ref).max()))
        assert np.array_equal(ys, plan.fused_dequant_gemv(dp, ds, dx, split_k=split).cpu().numpy())


@pytest.mark.gpu
def test_gptq_awq_argument_errors(cuda):
    from oxicuda_b200 import _lib as L
    from oxicuda_b200._lib import default_handle, ptr
    h = default_handle()
    p = torch.zeros(64, dtype=torch.int32, device=cuda)
    f = torch.zeros(640, dtype=torch.float32, device=cuda)
    with pytest.raises(L.InvalidArgument, match="bits must be"):
        h.call("b2q_wq_dequantize", ptr(p), ptr(f), None, 4, 32, 32, 5, ptr(f), L.OUT_F32)
    with pytest.raises(L.InvalidArgument, match="divisible"):
        h.call("b2q_wq_dequantize", ptr(p), ptr(f), None, 4, 48, 32, 4, ptr(f), L.OUT_F32)
    with pytest.raises(L.InvalidDimension):
        h.call("b2q_wq_dequantize", ptr(p), ptr(f), None, 0, 32, 32, 4, ptr(f), L.OUT_F32)
    with pytest.raises(L.InvalidArgument, match="multiple of the 10 values"):
        h.call("b2q_fused_dequant_gemv_f32", ptr(p), ptr(f), None, ptr(f), 2, 128, 64, 3, 1, ptr(f))
    with pytest.raises(L.InvalidArgument, match="split_k"):
        h.call("b2q_fused_dequant_gemv_f32", ptr(p), ptr(f), None, ptr(f), 2, 64, 32, 4, 3, ptr(f))
    with pytest.raises(L.InvalidArgument, match="AWQ bits"):
        h.call("b2q_awq_quantize_f32", ptr(f), ptr(f), ptr(f), 2, 64, 32, 2, ptr(p), None)
