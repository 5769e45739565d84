"""CPU: the oracle against every known-answer vector the reference's own tests hold for this path
(tests/golden/reference_kat.json, transcribed with file:line citations)."""
import math

import numpy as np
import pytest

CLASS_NAMES = ["SmallSquare", "LargeSquare", "SkinnyM", "SkinnyN", "SkinnyK", "General"]


def test_minmax_calibration_pins(oracle, kat):
    k = kat["minmax"]
    c = k["symmetric_calibrate_scale"]
    s, z, st = oracle.minmax_calibrate(c["x"], 1, len(c["x"]), c["bits"], c["scheme"])
    assert st == 0 and abs(s[0] - c["scale"]) < c["eps"] and z[0] == c["zp"]
    c = k["asymmetric_calibrate_scale_zp"]
    s, z, st = oracle.minmax_calibrate(c["x"], 1, len(c["x"]), c["bits"], c["scheme"])
    assert st == 0 and abs(s[0] - c["scale"]) < c["eps"] and z[0] == c["zp"]
    c = k["per_group_calibrate"]
    s, z, st = oracle.minmax_calibrate(c["x"], len(c["x"]) // c["group"], c["group"], c["bits"], 0)
    assert len(s) == c["n_scales"]
    c = k["calibrate_2d_per_row"]
    s, z, st = oracle.minmax_calibrate(c["x"], c["rows"], c["cols"], 8, 0)
    assert len(s) == 2 and s[1] > s[0]


def test_minmax_round_trips(oracle, kat):
    c = kat["minmax"]["symmetric_round_trip_low_error"]
    n = c["n"]
    t = (np.arange(n, dtype=np.float32) / np.float32(n - 1)) * 2 - 1
    s, z, _ = oracle.minmax_calibrate(t, 1, n, 8, 0)
    codes = oracle.minmax_quantize(t, 1, n, s, z, 8, 0)
    assert codes.min() >= -128 and codes.max() <= 127
    assert np.abs(oracle.minmax_dequantize(codes, 1, n, s, z) - t).max() < c["max_err"]
    c = kat["minmax"]["grouped_round_trip"]
    t = np.arange(c["n"], dtype=np.float32) * np.float32(c["step"])
    g = c["group"]
    s, z, _ = oracle.minmax_calibrate(t, c["n"] // g, g, c["bits"], 0)
    codes = oracle.minmax_quantize(t, c["n"] // g, g, s, z, c["bits"], 0)
    assert np.abs(oracle.minmax_dequantize(codes, c["n"] // g, g, s, z) - t).max() < c["max_err"]


def test_fp8_codec_pins(oracle, kat):
    k = kat["fp8_codec"]
    codes, bad = oracle.fp8_encode(np.array(k["e4m3_zero"]["x"], np.float32), 0, 0)
    assert bad == -1 and list(codes) == k["e4m3_zero"]["codes"]
    for name, fmt in (("e4m3_round_trip_basic", 0), ("e5m2_round_trip_basic", 1)):
        x = np.array(k[name]["x"], np.float32)
        dec = oracle.fp8_decode(oracle.fp8_encode(x, fmt, 0)[0], fmt, 0)
        assert (np.abs(x - dec) / np.maximum(np.abs(x), 1e-6)).max() < k[name]["rel_err"]
    dec = oracle.fp8_decode(oracle.fp8_encode([k["e4m3_saturates_large_values"]["x"]], 0, 0)[0], 0, 0)
    assert 0 < dec[0] <= k["e4m3_saturates_large_values"]["max"]
    assert oracle.fp8_encode([1.0, float("nan")], 0, 0)[1] == 1
    assert oracle.fp8_encode([float("inf")], 0, 0)[1] == 0
    data = np.arange(256, dtype=np.float32) / np.float32(128.0) - 1
    dec = oracle.fp8_decode(oracle.fp8_encode(data, 0, 0)[0], 0, 0)
    assert float(((data - dec) ** 2).sum() / 256) < k["mse_within_tolerance"]["mse"]
    for fmt, key in ((0, "e4m3"), (1, "e5m2")):
        for code, val in k["type_decode"][key].items():
            for mode in (0, 1):
                assert oracle.fp8_decode([int(code, 16)], fmt, mode)[0] == val


def test_fp8_rne_pins(oracle, kat):
    k = kat["fp8_rne"]
    for name in ("e4m3_encode_known_patterns", "e4m3_flush_to_zero", "e4m3_saturation"):
        codes, _ = oracle.fp8_encode(np.array(k[name]["x"], np.float32), 0, 1)
        assert list(codes) == k[name]["codes"], name
    assert oracle.fp8_decode([0x7E], 0, 1)[0] == k["e4m3_saturation"]["decode_0x7E"]
    codes, _ = oracle.fp8_encode(np.array(k["e4m3_subnormal_boundary"]["x"], np.float32), 0, 1)
    assert [c & 0x7F for c in codes] == k["e4m3_subnormal_boundary"]["codes_low7"]
    codes, _ = oracle.fp8_encode(np.array(k["e4m3_round_to_nearest_even"]["x"], np.float32), 0, 1)
    assert [c & 7 for c in codes] == k["e4m3_round_to_nearest_even"]["mantissa"]
    # the encoder never emits the NaN pattern (sweep of the reference's saturation test)
    v = np.clip(np.arange(256, dtype=np.float32) * np.float32(1.9) - 240, -448, 448)
    for mode in (0, 1):
        codes, _ = oracle.fp8_encode(v, 0, mode)
        assert not np.any((codes & 0x7F) == 0x7F)


def test_fp8_rne_round_trips_every_code(oracle):
    """IEEE decode then RNE encode is the identity on every finite E4M3/E5M2 code."""
    for fmt in (0, 1):
        codes = np.arange(256, dtype=np.uint8)
        dec = oracle.fp8_decode(codes, fmt, 1)
        ok = np.isfinite(dec)
        enc, _ = oracle.fp8_encode(dec[ok], fmt, 1)
        want = codes[ok].copy()
        assert np.array_equal(enc, want)


def test_fp8_ref_codec_derived_vectors(oracle):
    """Behaviour that only the reference's code pins (truncation, exp-15 saturation, halved subnormals)."""
    x = np.array([1.0, 1.95, -1.95, 0.5, 255.9, 256.0, 300, 448, 1000, 2**-6, 2**-7, 0.01, 2**-9, 2**-10, 1e-4], np.float32)
    codes, _ = oracle.fp8_encode(x, 0, 0)
    assert list(codes) == [0x38, 0x3F, 0xBF, 0x30, 0x77, 0x7E, 0x7E, 0x7E, 0x7E, 0x08, 0x02, 0x02, 0, 0, 0]
    dec = oracle.fp8_decode(np.array([0x3F, 0x77, 0x7E, 0x08, 0x02], np.uint8), 0, 0)
    assert list(dec) == [1.875, 240.0, 448.0, 2.0**-6, 0.01953125]


def test_fp4_pins(oracle, kat):
    k = kat["fp4"]
    c = k["fp4_e2m1_roundtrip_accuracy"]
    x = np.array(c["x"], np.float32)
    rec = oracle.fp4_dequantize(oracle.fp4_quantize(x, 0), 0)
    assert np.all(np.abs(x - rec) <= np.abs(x) * c["tol_rel"] + c["tol_abs"])
    assert np.array_equal(rec, x)      # all of them are exactly representable
    c = k["fp4_int4_roundtrip"]
    x = np.array(c["x"], np.float32)
    assert np.abs(oracle.fp4_dequantize(oracle.fp4_quantize(x, 1), 1) - x).max() < c["tol_abs"]
    for case in k["block_scale_rules"]["cases"]:
        _, s = oracle.fp4_block_quantize(np.full(32, case["fill"], np.float32), 32, 0, 0)
        assert abs(s[0] - case["scale"]) < 1e-6
    for n, want in k["block_scale_rules"]["num_scales"].items():
        _, s = oracle.fp4_block_quantize(np.ones(int(n), np.float32), 32, 0, 0)
        assert len(s) == want
    # element 2i sits in the low nibble
    assert list(oracle.fp4_quantize(np.array([1.0, 6.0], np.float32), 0)) == [2 | (7 << 4)]


def test_e2m1_derived_vectors(oracle):
    cases = {0.3: 0, 0.5: 0, 0.74: 0, 0.75: 1, 0.99: 1, 1.0: 2, 1.49: 2, 1.5: 3, 1.99: 3, 2.0: 4, 2.99: 4, 3.0: 5,
             3.99: 5, 4.0: 6, 5.99: 6, 6.0: 7, 7.0: 7, -2.5: 12, -0.3: 8, -0.0: 0, 0.0: 0}
    for v, code in cases.items():
        assert oracle.fp4_quantize_one(v, 0) == code, v
    assert oracle.fp4_quantize_one(float("nan"), 0) == 7
    vals = [oracle.fp4_dequantize_one(c, 0) for c in range(16)]
    assert vals[:8] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0] and vals[8:] == [-v for v in vals[:8]]
    # neighbours of the thresholds that change the exponent
    for t in (0.5, 1.0, 2.0, 4.0):
        below = float(np.nextafter(np.float32(t), np.float32(0)))
        assert oracle.fp4_quantize_one(below, 0) < oracle.fp4_quantize_one(t, 0) or t == 0.5


def test_e8m0_rule(oracle):
    """parity unpinned (E8M0 is absent from the reference): smallest power of two >= absmax/6."""
    assert oracle.e8m0_from_absmax(0.0) == 127
    assert oracle.e8m0_from_absmax(6.0) == 127
    assert oracle.e8m0_from_absmax(6.0001) == 128
    assert oracle.e8m0_from_absmax(12.0) == 128
    assert oracle.e8m0_from_absmax(3.0) == 126
    rng = np.random.default_rng(3)
    for a in np.abs(rng.standard_normal(200).astype(np.float32)) * 0.1 + 1e-6:
        e = oracle.e8m0_from_absmax(float(a)) - 127
        s = np.float32(a) / np.float32(6.0)
        assert 2.0**e >= s > 2.0 ** (e - 1)
    x = (rng.standard_normal(4096) * 0.02).astype(np.float32)
    packed, sc = oracle.fp4_block_quantize(x, 32, 0, 1)
    deq = oracle.fp4_block_dequantize(packed, sc, x.size, 32, 0)
    blk_max = np.abs(x).reshape(-1, 32).max(1).repeat(32)
    assert np.all(np.abs(deq - x) <= blk_max * 0.34 + 1e-12)     # truncation onto the E2M1 grid under a 2x scale


def test_tile_pins(oracle, kat):
    k = kat["tiles"]
    for m, n, kk, name in k["classify_workload"]["cases"]:
        assert CLASS_NAMES[oracle.classify_workload(m, n, kk)] == name
    c = k["fp8_blackwell_large_square"]
    t = oracle.tile_config(0, *c["mnk"])
    assert (t[0], t[1], t[5]) == (c["tile_m"], c["tile_n"], c["stages"])
    c = k["fp8_blackwell_skinny_m"]
    assert oracle.tile_config(0, *c["mnk"])[:2] == (c["tile_m"], c["tile_n"])
    c = k["fp4_tile_blackwell_skinny_m"]
    assert oracle.tile_config(1, *c["mnk"])[:2] == (c["tile_m"], c["tile_n"])
    c = k["fp4_tile_blackwell_large"]
    assert oracle.tile_config(1, *c["mnk"])[:3] == (c["tile_m"], c["tile_n"], c["tile_k"])
    t = oracle.tile_config(2, 512, 512, 512)
    assert (t[2], t[5]) == (k["int8_tile_hopper_plus"]["tile_k"], k["int8_tile_hopper_plus"]["stages"])
    assert oracle.fp8_split_k(16, 16, 65536) == 8 and oracle.fp8_split_k(4096, 4096, 4096) == 1


def test_llm_int8_pins(oracle, kat):
    k = kat["llm_int8"]
    c = k["detects_outlier_column"]
    r = oracle.llm_int8_matmul(c["x"], np.ones(5 * 2, np.float32), c["samples"], 2, c["cols"], 6.0, True)
    assert list(np.nonzero(r["outlier_mask"])[0]) == c["outliers"]
    c = k["no_outliers_when_below_threshold"]
    r = oracle.llm_int8_matmul(c["x"], np.ones(5 * 2, np.float32), c["samples"], 2, c["cols"], 6.0, True)
    assert r["n_outliers"] == 0
    c = k["matmul_matches_fp32_when_no_outliers"]
    x = np.array(c["x"], np.float32).reshape(c["samples"], c["cols"])
    w = np.array(c["w"], np.float32).reshape(c["rows"], c["cols"])
    r = oracle.llm_int8_matmul(x, w, c["samples"], c["rows"], c["cols"], 6.0, True)
    assert r["n_outliers"] == 0
    ref = (x.astype(np.float64) @ w.astype(np.float64).T).reshape(-1)
    rmse = math.sqrt(float(((r["output"] - ref) ** 2).mean()))
    assert rmse < c["rmse_frac"] * max(np.abs(ref).max(), 1e-6)
    c = k["outlier_fraction_reported"]
    r = oracle.llm_int8_matmul(c["x"], c["w"], c["samples"], c["rows"], c["cols"], 6.0, True)
    assert abs(r["n_outliers"] / c["cols"] - c["fraction"]) < 1e-6


def test_distfp8_pins(oracle, kat):
    k = kat["distfp8"]
    for name in ("zero_quantizes_to_zero", "max_quantized_value_is_127", "negative_packs_as_twos_complement"):
        x = np.array(k[name]["x"], np.float32)
        q, _ = oracle.distfp8_quantize_block(x, x.size)
        assert list(q) == k[name]["q"], name
    c = k["block_scales_shape"]
    _, s = oracle.distfp8_quantize_block(np.ones(c["n"], np.float32), c["block"])
    assert len(s) == c["n_scales"]
    c = k["block_all_zeros_scale_is_zero"]
    q, s = oracle.distfp8_quantize_block(np.array(c["x"], np.float32), c["block"])
    assert s[0] == 0.0 and s[1] > 0.0 and list(q[:4]) == [0, 0, 0, 0]


def test_tensor_parallel_pins(oracle, kat):
    c = kat["tensor_parallel"]["ring_all_reduce_sum"]
    # RowLinear::all_reduce == sum in rank order: identity weights, one input column per rank
    ranks = np.array(c["ranks"], np.float32)            # [tp][out]
    tp, out_f = ranks.shape
    x = np.ones((1, tp), np.float32)
    w = ranks.T.copy()                                  # [out x in], in = tp, one column per rank
    got = oracle.row_linear(x, w, None, 1, tp, out_f, tp)
    assert list(got[0]) == c["sum"]
    # identity TP round trip gives ones (crates/oxicuda-dist-infer/src/lib.rs:139-184)
    n = 8
    eye = np.eye(n, dtype=np.float32)
    xin = np.ones((2, n), np.float32)
    for tp in (1, 2, 4):
        mid = oracle.column_linear(xin, eye, None, 2, n, n, tp)
        assert np.array_equal(oracle.row_linear(mid, eye, None, 2, n, n, tp), xin)


def test_nf4_round_trip(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(64 * 8).astype(np.float32)
    packed, am = oracle.nf4_encode(x, 64)
    dec = oracle.nf4_decode(packed, am, 64)
    assert np.abs(dec - x).max() <= np.abs(x).max() * 0.16
    lut_hit = oracle.nf4_decode(oracle.nf4_encode(np.array([1.0, -1.0] * 32, np.float32), 64)[0], np.ones(1, np.float32), 64)
    assert np.array_equal(lut_hit, np.array([1.0, -1.0] * 32, np.float32))


def _kv_lcg(n, seed, amp):
    from tests.golden.make_reference_kat import lcg
    return np.array(lcg(n, seed, amp), np.float32)


def _kv_rel_err(a, b):
    """rel_err of crates/oxicuda-quant/src/scheme/kv_cache.rs:298-306"""
    return float(np.abs(a - b).sum() / max(np.abs(a).sum(), 1e-8))


def test_kv_cache_pins(oracle, kat):
    k = kat["kv_cache"]
    for name in ("int8_per_token_round_trip", "int8_per_channel_round_trip", "int4_round_trip_coarser_but_bounded"):
        c = k[name]
        x = _kv_lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"])
        codes, s, z = oracle.kv_cache_quantize(x, c["n_tokens"], c["head_dim"], c["bits"], c["axis"])
        assert len(s) == len(z) == c["n_groups"] and int(codes.max()) <= (1 << c["bits"]) - 1
        deq = oracle.kv_cache_dequantize(codes, c["n_tokens"], c["head_dim"], c["axis"], s, z)
        assert _kv_rel_err(x, deq) < c["rel_err"], name
    c = k["per_channel_beats_per_token_on_key_outliers"]
    x = _kv_lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"]).reshape(c["n_tokens"], c["head_dim"])
    x[:, c["outlier_col"]] = np.float32(c["outlier_base"]) + np.arange(c["n_tokens"], dtype=np.float32) * np.float32(c["outlier_step"])
    errs = []
    for axis in (1, 0):
        codes, s, z = oracle.kv_cache_quantize(x, c["n_tokens"], c["head_dim"], 8, axis)
        errs.append(_kv_rel_err(x.reshape(-1), oracle.kv_cache_dequantize(codes, c["n_tokens"], c["head_dim"], axis, s, z)))
    assert errs[0] < errs[1]
    c = k["append_token_grows_cache"]           # append_token == the per-token rule on one more row
    x = _kv_lcg(c["n_tokens"] * c["head_dim"], c["seed"], c["amp"])
    row = _kv_lcg(c["head_dim"], c["row_seed"], c["amp"])
    codes, s, z = oracle.kv_cache_quantize(x, c["n_tokens"], c["head_dim"], 8, 0)
    rc, rs, rz = oracle.kv_cache_quantize(row, 1, c["head_dim"], 8, 0)
    both = oracle.kv_cache_quantize(np.concatenate([x, row]), c["n_tokens"] + 1, c["head_dim"], 8, 0)
    assert np.array_equal(np.concatenate([codes, rc]), both[0]) and np.array_equal(np.concatenate([s, rs]), both[1])
    assert _kv_rel_err(row, oracle.kv_cache_dequantize(rc, 1, c["head_dim"], 0, rs, rz)) < c["rel_err"]


def test_kv_quant_token_pins(oracle, kat):
    k = kat["kv_quant"]
    c = k["asymmetric_endpoints_exact"]
    x = np.array(c["x"], np.float32)
    codes, s, z = oracle.kv_quantize_tokens(x, 1, x.size, 8, False)
    r = oracle.kv_dequantize_tokens(codes, 1, x.size, s, z)
    assert z[0] == c["zero_point"] and abs(r[0] - x[0]) < c["tol"] and abs(r[-1] - x[-1]) < c["tol"]
    assert codes.min() == k["q_range_signed_and_unsigned"]["asym8"][0] and codes.max() == k["q_range_signed_and_unsigned"]["asym8"][1]
    c = k["symmetric_zero_point_is_zero"]
    x = np.array(c["x"], np.float32)
    codes, s, z = oracle.kv_quantize_tokens(x, 1, x.size, 8, True)
    r = oracle.kv_dequantize_tokens(codes, 1, x.size, s, z)
    assert z[0] == c["zero_point"] and float(((x - r).astype(np.float64) ** 2).mean()) < c["mse"]
    assert [int(codes.min()), int(codes.max())] == k["q_range_signed_and_unsigned"]["sym8"]
    c = k["constant_vector_zero_error"]
    x = np.array(c["x"], np.float32)
    codes, s, z = oracle.kv_quantize_tokens(x, 1, x.size, 8, False)
    assert np.abs(oracle.kv_dequantize_tokens(codes, 1, x.size, s, z) - x).max() < c["tol"]
    c = k["mse_decreases_with_precision_on_smooth_signal"]
    x = np.cos(np.arange(c["n"], dtype=np.float32) * np.float32(c["step"])).astype(np.float32)
    mse = []
    for bits in (4, 8):
        codes, s, z = oracle.kv_quantize_tokens(x, 1, x.size, bits, False)
        assert codes.max() <= (1 << bits) - 1 and codes.min() >= 0
        mse.append(float(((x - oracle.kv_dequantize_tokens(codes, 1, x.size, s, z)).astype(np.float64) ** 2).mean()))
    assert mse[1] <= mse[0] and mse[1] < c["mse8"]


def test_rms_norm_pins(oracle, kat):
    c = kat["rms_norm"]["formula"]
    y = oracle.rms_norm(c["x"], np.ones(len(c["x"]), np.float32), 1, len(c["x"]), c["eps"])
    assert np.abs(y - np.array(c["approx"], np.float32)).max() < c["tol"]
    c = kat["rms_norm"]["uniform_input"]
    y = oracle.rms_norm(c["x"], np.ones(len(c["x"]), np.float32), 1, len(c["x"]), c["eps"])
    assert np.abs(y - c["y"]).max() < c["tol"]
    # fused residual form: the norm of (residual + x), residual updated in place
    x = np.array([1.0, -2.0, 0.5, 4.0], np.float32); res = np.array([0.5, 0.5, -1.0, 2.0], np.float32)
    g = np.array([1.0, 2.0, 0.5, 1.5], np.float32)
    y, new_res = oracle.rms_norm(x, g, 1, 4, 1e-6, residual=res)
    assert np.array_equal(new_res, x + res) and np.array_equal(y, oracle.rms_norm(x + res, g, 1, 4, 1e-6))


class DnnLcg:
    """Lcg of crates/oxicuda-dnn/src/gpu_tests/mod.rs:169-189."""

    def __init__(self, seed):
        self.s = seed

    def next_u32(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return self.s >> 32

    def range_f32(self, lo, hi):
        return np.float32(lo + (hi - lo) * (self.next_u32() / 4294967296.0))


def test_dnn_quantize_pins(oracle, kat):
    """The oracle run through the assertions of the reference's GPU tests (gpu_tests/quantize.rs:184-325, :503-554)."""
    import torch
    k = kat["dnn_quantize"]
    c = k["int8_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    q, s = oracle.dnn_quantize_to_int8(data)
    assert s[0] == max(np.float32(np.abs(data).max()) / np.float32(127.0), np.float32(1e-12))
    assert np.array_equal(q, np.rint(np.clip(data / s[0], -127.0, 127.0)).astype(np.int8))
    c = k["fp8_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    codes, s = oracle.dnn_quantize_to_fp8(data)
    assert s[0] == max(np.float32(np.abs(data).max()) / np.float32(448.0), np.float32(1e-12))
    scaled = torch.from_numpy(np.clip(data / s[0], -448.0, 448.0).astype(np.float32))
    assert np.array_equal(codes, scaled.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    c = k["fp8_dequantize_numeric"]
    b = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(b).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    ref[0x7F], ref[0xFF] = 480.0, -480.0
    assert np.array_equal(oracle.dnn_dequantize_from_fp8(b, c["scale"]), ref * np.float32(c["scale"]))
    c = k["block_quantize_numeric"]
    lcg = DnnLcg(c["seed"])
    data = np.array([lcg.range_f32(c["lo"], c["hi"]) for _ in range(c["n"])], np.float32)
    out, sc = oracle.dnn_quantize_block_scaled(data, c["block"])
    assert np.array_equal(sc, np.maximum(np.abs(data).reshape(-1, c["block"]).max(axis=1) / np.float32(6.0), np.float32(1e-12)))
    assert np.array_equal(out, np.clip(np.rint(np.clip(data / np.repeat(sc, c["block"]), -6.0, 6.0)).astype(np.int32) + 6, 0, 255))
    c = k["block_int8_gptq_dequant_precision"]
    deq = oracle.block_int8_dequantize(np.array(c["data"], np.int8), [c["scale"]], 3)
    assert np.abs(deq - np.array(c["expected"], np.float32)).max() < c["tol"]
    c = k["block_int8_round_trip"]
    x = ((np.arange(c["n"], dtype=np.float32) - np.float32(c["offset"])) / np.float32(c["div"])).astype(np.float32)
    q, sc = oracle.block_int8_quantize(x, c["block"])
    assert np.abs(oracle.block_int8_dequantize(q, sc, c["block"]) - x).max() < c["tol"] and len(sc) == 4
    c = k["block_int8_non_multiple_len"]
    q, sc = oracle.block_int8_quantize(np.arange(c["n"], dtype=np.float32), c["block"])
    assert len(sc) == c["num_blocks"] and len(q) == c["n"]
    c = k["fp4_block_quantizer"]
    assert oracle.block_absmax_scale(np.zeros(32, np.float32), 32)[0] == c["zeros_scale"]
    assert oracle.block_absmax_scale(np.full(32, 12.0, np.float32), 32)[0] == c["twelve_scale"]
    for n, want in c["num_scales"]:
        assert len(oracle.block_absmax_scale(np.ones(n, np.float32), 32)) == want


def test_int4_pins(oracle, kat):
    k = kat["int4"]
    v = k["pack_unpack_roundtrip"]["values"]
    packed, st = oracle.pack_int4(v)
    assert st == 0 and packed.size == 1 and list(oracle.unpack_int4(packed)) == v
    assert oracle.pack_int4(k["pack_wrong_length"]["values"])[1] == 1
    assert oracle.pack_int4(k["pack_out_of_range"]["values"])[1] == 2 + 7
    for word, vals in k["unpack_words"]["cases"]:
        assert list(oracle.unpack_int4([word])) == vals
    # the GEMM against a float64 statement of dequantize-then-multiply on a small case
    rng = np.random.default_rng(41)
    M, N, K, group = 5, 3, 64, 32
    vals = rng.integers(-8, 8, (M, K)).astype(np.int8)
    packed, _ = oracle.pack_int4(vals)
    scales = (rng.uniform(0.01, 0.1, (M, K // group))).astype(np.float16)
    b = rng.standard_normal((K, N)).astype(np.float32)
    c = oracle.gemm_int4(packed, scales, b, M, N, K, group)
    w = vals.astype(np.float64) * np.repeat(scales.astype(np.float64), group, axis=1)
    assert np.allclose(c, w @ b.astype(np.float64), rtol=1e-5, atol=1e-5)
