"""CPU: the C-ABI library loads without a GPU, exports every symbol the header declares, and the
host-side logic (tile heuristics, argument validation, error mapping) behaves like the reference."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CLASS_NAMES = ["SmallSquare", "LargeSquare", "SkinnyM", "SkinnyN", "SkinnyK", "General"]


def _header_symbols():
    text = (ROOT / "include" / "b2q.h").read_text()
    return sorted(set(re.findall(r"\b(b2q_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(libb2q):
    from oxicuda_b200 import _lib
    names = _header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(libb2q, n), f"{n} is declared in include/b2q.h but missing from libb2q.so"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_no_cpu_fallback_without_device(libb2q):
    import torch
    from oxicuda_b200 import _lib
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(_lib.B2qError):
        _lib.Handle(0)


def test_null_handle_is_rejected(libb2q):
    assert libb2q.b2q_check(None) == 8
    assert libb2q.b2q_gemm_fp8(None, None, None, 1, 1, 16, 0, None, 0, None, 0, None, 0) == 8
    assert libb2q.b2q_last_error(None) == b"null handle"


def test_tile_heuristics_match_reference_pins(libb2q, kat, oracle):
    from oxicuda_b200 import blas
    k = kat["tiles"]
    for m, n, kk, name in k["classify_workload"]["cases"]:
        assert blas.classify_workload(m, n, kk).name == name
    c = k["fp8_blackwell_large_square"]
    t = blas.Fp8Config.tile_config(*c["mnk"])
    assert (t.tile_m, t.tile_n, t.stages) == (c["tile_m"], c["tile_n"], c["stages"])
    c = k["fp8_blackwell_skinny_m"]
    t = blas.Fp8Config.tile_config(*c["mnk"])
    assert (t.tile_m, t.tile_n) == (c["tile_m"], c["tile_n"])
    c = k["fp4_tile_blackwell_skinny_m"]
    t = blas.select_fp4_tile(*c["mnk"])
    assert (t.tile_m, t.tile_n) == (c["tile_m"], c["tile_n"])
    c = k["fp4_tile_blackwell_large"]
    t = blas.select_fp4_tile(*c["mnk"])
    assert (t.tile_m, t.tile_n, t.tile_k) == (c["tile_m"], c["tile_n"], c["tile_k"])
    t = blas.int8_tile_config(512, 512, 512)
    assert (t.tile_k, t.stages) == (k["int8_tile_hopper_plus"]["tile_k"], k["int8_tile_hopper_plus"]["stages"])
    # the library and the oracle agree on a sweep of shapes
    for dtype in (0, 1, 2):
        for m in (1, 8, 64, 127, 128, 1024, 4096):
            for n in (1, 64, 128, 1000, 4096, 14336):
                for kk in (1, 32, 63, 64, 4096, 40000):
                    t = blas._ref_tile(dtype, m, n, kk)
                    assert t.as_tuple() == oracle.tile_config(dtype, m, n, kk), (dtype, m, n, kk)
                    assert blas.classify_workload(m, n, kk).value == oracle.classify_workload(m, n, kk)
                    assert blas.Fp8Config.compute_split_k(m, n, kk) == oracle.fp8_split_k(m, n, kk)


def test_zero_dimension_is_invalid_dimension(libb2q):
    from oxicuda_b200 import _lib, blas
    with pytest.raises(_lib.InvalidDimension):
        blas.Fp8Config.tile_config(0, 4, 4)
    with pytest.raises(_lib.InvalidDimension):
        blas.select_tile("fp8", 4, 0, 4)


def test_static_tile_table(libb2q):
    from oxicuda_b200 import blas
    t, kid = blas.select_tile("fp8", 4096, 4096, 4096)
    assert kid == 4 and (t.tile_m, t.tile_n, t.tile_k) == (256, 256, 128)      # two-CTA pair tiles
    t, kid = blas.select_tile("fp8", 128, 4096, 4096)
    assert kid in (1, 2) and t.tile_m == 128 and t.tile_n in (128, 256)
    t, kid = blas.select_tile("fp8", 8, 4096, 4096)
    assert kid == 5 and t.tile_n == 16                # decode-sized: tensor-core GEMV over the codes
    t, kid = blas.select_tile("fp8", 40, 4096, 4096)
    assert kid == 6                                   # between the GEMV and a 128-row tile: weight-stationary tcgen05 kernel
    t, kid = blas.select_tile("fp8", 40, 4096, 4000)
    assert kid == 0                                   # K not a multiple of 128 (nor of 16): SIMT path
    t, kid = blas.select_tile("fp8", 4096, 4096, 4100)
    assert kid == 0                                   # row pitch TMA cannot take
    t, kid = blas.select_tile("fp4", 1, 4096, 4096)
    assert kid == 3 and t.tile_m == 8 and t.tile_n == 128
    t, kid = blas.select_tile("fp4", 32, 1024, 4096)
    assert kid == 3 and t.tile_m == 32 and t.tile_n == 64


def test_python_side_validation_mirrors_reference_errors(libb2q, kat):
    import torch
    from oxicuda_b200 import _lib, blas, quant
    q = quant.MinMaxQuantizer.int8_symmetric()
    with pytest.raises(_lib.EmptyInput):
        q.calibrate(torch.empty(0))
    with pytest.raises(_lib.EmptyInput):
        q.calibrate_2d(torch.empty(0), 0, 4)
    with pytest.raises(_lib.DimensionMismatch):
        q.calibrate_2d(torch.empty(0), 2, 0)
    for bad in kat["llm_int8"]["config_validation"]["bad"]:
        with pytest.raises(_lib.InvalidConfig):
            quant.LlmInt8Config.new(float(bad), True)
    assert quant.LlmInt8Config.new(6.0, True).threshold == 6.0
    cfg = quant.LlmInt8Config()
    assert cfg.threshold == 6.0 and cfg.row_wise_activations
    lq = quant.LlmInt8Quantizer()
    with pytest.raises(_lib.EmptyInput):
        lq.matmul(torch.empty(0), torch.ones(4), 1, 1, 4)
    with pytest.raises(_lib.DimensionMismatch):
        lq.matmul(torch.ones(10), torch.ones(4), 3, 1, 4)
    for a, b in kat["fp4"]["packed_fp4_overflow_rejected"]["bad"]:
        with pytest.raises(_lib.InvalidArgument):
            blas.PackedFp4.pack(a, b)
    for a in range(16):
        for b in range(16):
            assert blas.PackedFp4.unpack(blas.PackedFp4.pack(a, b)) == (a, b)
    for bs in kat["fp4"]["block_size_validation"]["invalid"]:
        with pytest.raises(_lib.InvalidArgument):
            blas.MicroScalingConfig(block_size=bs).validate()
    for bs in kat["fp4"]["block_size_validation"]["valid"]:
        blas.MicroScalingConfig(block_size=bs).validate()
    p = quant.QuantParams(torch.ones(1), torch.zeros(1, dtype=torch.int32), 8, quant.QuantScheme.Symmetric)
    assert (p.q_max(), p.q_min()) == (kat["minmax"]["q_max_q_min_int8"]["q_max"], kat["minmax"]["q_max_q_min_int8"]["q_min"])


def test_kv_cache_host_side_validation(libb2q, kat):
    """Config and shape checks of the KV-cache mirrors fail before anything touches a device, with the reference's errors."""
    import torch
    from oxicuda_b200 import _lib
    from oxicuda_b200.kv_cache import (KvAxis, KvCacheConfig, KvCacheQuantizer, KvQuantConfig, QuantizedKvCache, quantize_tokens)
    c = kat["kv_cache"]["config_validates_bits"]
    for bits in c["ok"]:
        KvCacheConfig.new(bits, KvAxis.PerToken)
    for bits in c["bad"]:
        with pytest.raises(_lib.InvalidBitWidth):
            KvCacheConfig.new(bits, KvAxis.PerToken)
    assert KvCacheConfig.keys_int8().axis == KvAxis.PerChannel and KvCacheConfig.values_int8().axis == KvAxis.PerToken
    q = KvCacheQuantizer(KvCacheConfig.values_int8())
    with pytest.raises(_lib.EmptyInput):
        q.quantize(torch.empty(0), 0, 0)
    with pytest.raises(_lib.DimensionMismatch):
        q.quantize(torch.ones(10), 3, 4)
    cache = QuantizedKvCache(torch.zeros(32, dtype=torch.uint8), torch.ones(4), torch.zeros(4), 4, 8, 4, KvAxis.PerToken)
    c = kat["kv_cache"]["packed_bytes_reflects_bit_width"]
    assert cache.packed_bytes() == c["bits4_bytes"] and cache.n_groups() == 4
    cache.bits = 8
    assert cache.packed_bytes() == c["bits8_bytes"]
    with pytest.raises(_lib.DimensionMismatch):
        q.append_token(cache, torch.ones(5))
    cache.axis = KvAxis.PerChannel
    with pytest.raises(_lib.InvalidConfig):
        q.append_token(cache, torch.ones(8))
    r = kat["kv_quant"]["q_range_signed_and_unsigned"]
    assert list(KvQuantConfig.new(8, False).q_range()) == r["asym8"] and list(KvQuantConfig.new(8, True).q_range()) == r["sym8"]
    assert list(KvQuantConfig.new(4, False).q_range()) == r["asym4"] and KvQuantConfig.int8() == KvQuantConfig(8, False)
    with pytest.raises(_lib.InvalidConfig):
        KvQuantConfig.new(3, False)
    with pytest.raises(_lib.InvalidConfig):
        quantize_tokens(torch.empty(0, 4), KvQuantConfig.int8())


def test_rank_coordinates_and_shard_ranges(libb2q):
    from oxicuda_b200 import _lib
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, column_shard_rows, row_shard_cols
    cfg = ParallelismConfig(tp=2, sp=2, ep=2)
    assert cfg.world_size() == 8
    h = DistInferHandle(5, cfg)          # crates/oxicuda-dist-infer/src/handle.rs: tp=g%tp, sp=(g/tp)%sp, ep=g/(tp*sp)
    assert (h.tp_rank(), h.sp_rank(), h.ep_rank()) == (1, 0, 1)
    with pytest.raises(_lib.InvalidArgument):
        DistInferHandle(8, cfg)
    assert column_shard_rows(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert row_shard_cols(28672, 4, 1) == (7168, 14336)
    with pytest.raises(_lib.InvalidDimension):
        column_shard_rows(10, 3, 0)


def test_rust_bindings_cover_the_header(libb2q):
    """rust/b2q-sys/src/lib.rs is generated from include/b2q.h: it must declare exactly the symbols the header (and
    the ctypes table) declare, and be what the generator writes today."""
    import re
    import subprocess
    import sys
    from pathlib import Path
    from oxicuda_b200 import _lib
    root = Path(__file__).resolve().parent.parent
    src = (root / "rust" / "b2q-sys" / "src" / "lib.rs").read_text()
    names = set(re.findall(r"pub fn (b2q_[a-z0-9_]+)", src))
    assert names == set(_lib.SIGNATURES)
    before = src
    subprocess.run([sys.executable, str(root / "rust" / "b2q-sys" / "gen_ffi.py")], check=True, capture_output=True)
    assert (root / "rust" / "b2q-sys" / "src" / "lib.rs").read_text() == before
    # every item the wrapper crates take from the bindings exists there (the crates cannot be compiled here)
    declared = names | set(re.findall(r"pub const (B2Q_[A-Z0-9_]+)", src)) | set(re.findall(r"pub (?:type|struct) (b2q_[a-z0-9_]+)", src))
    for crate in ("oxicuda-blas-b200", "oxicuda-quant-b200", "oxicuda-dist-infer-b200", "oxicuda-dnn-b200"):
        used = set(re.findall(r"sys::([A-Za-z0-9_]+)", (root / "rust" / crate / "src" / "lib.rs").read_text()))
        assert used <= declared, (crate, sorted(used - declared))


def test_tp_boundary_plan(libb2q):
    """b2q_tp_plan (a pure host function): which row-parallel boundary a result of tokens x out_features takes."""
    def plan(tp, attached, tokens, out):
        mode, chunks = C.c_int(-1), C.c_int(-1)
        assert libb2q.b2q_tp_plan(tp, attached, C.c_int64(tokens), C.c_int64(out), C.byref(mode), C.byref(chunks)) == 0
        return mode.value, chunks.value
    assert plan(1, 1, 4096, 8192) == (0, 1)                      # one rank: no boundary
    assert plan(2, 1, 1, 8192) == (1, 1)                         # 32 KiB of fp32 partials: one-shot peer kernel
    assert plan(8, 1, 8, 8192) == (1, 1)                         # 256 KiB: still one-shot
    assert plan(2, 1, 64, 8192) == (2, 1)                        # 2 MiB: two-shot peer kernel
    assert plan(8, 1, 128, 8192) == (2, 1)                       # 4 MiB: the last two-shot size
    assert plan(8, 1, 4096, 8192) == (4, 1)                      # 64 MiB bf16: reduce-scatter inside the GEMM epilogue
    assert plan(2, 1, 2048, 768) == (4, 1)
    assert plan(2, 1, 4090, 8192)[0] == 3                        # rows do not split into 32-row blocks per rank: NCCL
    assert plan(8, 1, 8192, 8192)[0] == 3                        # 128 MiB: beyond the exchange buffer
    assert plan(2, 0, 64, 8192)[0] == 3 and plan(2, 0, 4096, 8192)[0] == 3   # no peer mappings: NCCL
    mode, chunks = C.c_int(), C.c_int()
    assert libb2q.b2q_tp_plan(0, 1, C.c_int64(1), C.c_int64(1), C.byref(mode), C.byref(chunks)) != 0
    assert libb2q.b2q_tp_plan(2, 1, C.c_int64(0), C.c_int64(8), C.byref(mode), C.byref(chunks)) != 0


def test_oracle_mlp_hidden_layouts(oracle):
    """oracle/api.py::swiglu_mlp_hidden: the interleaved statement equals the concatenated one up to where h is rounded
    (f32 gate | up and bf16 h against bf16 gate | up and f32 h), and interleave_rows128 is the layout of the header."""
    import numpy as np
    rng = np.random.default_rng(3)
    tokens, hidden, F = 5, 64, 256
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    wg = (rng.standard_normal((F, hidden)) * 0.1).astype(np.float32)
    wu = (rng.standard_normal((F, hidden)) * 0.1).astype(np.float32)
    xc, xs, _ = oracle.fp8_quantize_rows(x, tokens, hidden, 0, 1)
    gc, gs, _ = oracle.fp8_quantize_rows(wg, F, hidden, 0, 1)
    uc, us, _ = oracle.fp8_quantize_rows(wu, F, hidden, 0, 1)
    gc, uc = gc.reshape(F, hidden), uc.reshape(F, hidden)
    wi, si = oracle.interleave_rows128(gc, uc), oracle.interleave_rows128(gs, us)
    assert wi.shape == (2 * F, hidden) and si.shape == (2 * F,)
    assert np.array_equal(wi[:128], gc[:128]) and np.array_equal(wi[128:256], uc[:128]) and np.array_equal(wi[256:384], gc[128:])
    assert np.array_equal(si[128:256], us[:128])
    h_cat = oracle.swiglu_mlp_hidden(xc, xs, np.concatenate([gc, uc]), np.concatenate([gs, us]), tokens, hidden, F, False)
    h_int = oracle.swiglu_mlp_hidden(xc, xs, wi, si, tokens, hidden, F, True)
    scale = np.abs(h_cat).max()
    assert np.abs(h_cat - h_int).max() <= 2.0 ** -6 * scale      # a few bf16 roundings apart
    assert np.array_equal(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(h_int)).reshape(h_int.shape), h_int)   # h_int is bf16
