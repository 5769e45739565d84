"""GPU: the allocation-free FP8 quantizer entry point against the regular one.

Some users of this library cannot allocate device memory when they call it (their process has already
committed its whole memory budget, or they sit in a region where the allocator must stay untouched), so
b2q_fp8_quantize_rows_f32_noalloc keeps its reduction scratch in a fixed array inside the library instead
of a handle.  Called twice in a row, on different inputs, it must give exactly what b2q_fp8_quantize_rows_f32
gives: the shared array keeps the first call's contents, and the second call must not be disturbed by them.
This file sorts last so that a run stopping at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc(x, rows, cols, rounding, fmt=0, with_status=True):
    from oxicuda_b200 import _lib as L
    codes = torch.empty(rows * cols, dtype=torch.uint8, device=x.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    err = C.create_string_buffer(256)
    st = L.lib().b2q_fp8_quantize_rows_f32_noalloc(L.ptr(x), rows, cols, fmt, rounding, L.ptr(scales), L.ptr(codes),
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream),
                                                  L.ptr(status) if with_status else None, err, 256)
    return st, codes, scales, status, err.value.decode()


def test_no_alloc_entry_matches_regular_entry_twice(cuda):
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.quant import Fp8Codec
    g = torch.Generator(device=cuda).manual_seed(7)
    # call 1: many long slices (fills the shared scratch); call 2: one slice with a smaller absmax (stale keys would win)
    cases = [(64, 40000, 3.0, L.ROUND_REF), (1, 1 << 20, 0.02, L.ROUND_RNE), (1024, 96, 1.0, L.ROUND_RNE)]
    for rows, cols, sigma, rounding in cases:
        x = torch.randn(rows * cols, device=cuda, generator=g) * sigma
        st, codes, scales, status, msg = _noalloc(x, rows, cols, rounding)
        assert st == L.OK, msg
        ref_codes, ref_scales = Fp8Codec.e4m3("ref" if rounding == L.ROUND_REF else "rne").quantize_rows(x, rows, cols)
        torch.cuda.synchronize()
        assert torch.equal(scales.view(torch.int32), ref_scales.view(torch.int32)), (rows, cols)     # bit-exact
        assert torch.equal(codes, ref_codes), (rows, cols)
        assert int(status.item()) == 0


def test_no_alloc_entry_rejects_what_it_cannot_hold(cuda):
    from oxicuda_b200 import _lib as L
    x = torch.zeros(1025 * 4, device=cuda)
    st, _, _, _, msg = _noalloc(x, 1025, 4, L.ROUND_RNE)
    assert st == L.ERR_BUFFER_TOO_SMALL and "1024" in msg
    st, _, _, _, msg = _noalloc(x, 0, 4, L.ROUND_RNE)
    assert st == L.ERR_EMPTY_INPUT
    bad = torch.tensor([1.0, float("nan"), 2.0, 3.0], device=cuda)
    st, _, _, status, _ = _noalloc(bad, 1, 4, L.ROUND_RNE)
    torch.cuda.synchronize()
    assert st == L.OK and int(status.item()) == L.ERR_NON_FINITE_FP8


def test_no_alloc_entry_odd_shapes_formats_and_no_status_word(cuda):
    """The scalar fall-backs (a row length that is no multiple of 4, an input that is not 16-byte aligned), E5M2, and a call
    without a status word: the same bits as the regular entry point; without the status word a NaN goes unreported."""
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.quant import Fp8Codec
    g = torch.Generator(device=cuda).manual_seed(9)
    base = torch.randn(1 + 37 * 1001, device=cuda, generator=g)
    for x, rows, cols, fmt, name in ((base[1:], 37, 1001, 0, "e4m3"), (base[:36 * 1001], 36, 1001, 1, "e5m2")):
        # base[1:] starts 4 bytes past a 16-byte boundary: the scalar load path
        for with_status in (True, False):
            st, codes, scales, _, msg = _noalloc(x, rows, cols, L.ROUND_RNE, fmt, with_status)
            assert st == L.OK, msg
            codec = Fp8Codec.e4m3("rne") if fmt == 0 else Fp8Codec.e5m2("rne")
            ref_codes, ref_scales = codec.quantize_rows(x.contiguous(), rows, cols)
            torch.cuda.synchronize()
            assert torch.equal(scales.view(torch.int32), ref_scales.view(torch.int32)), name
            assert torch.equal(codes, ref_codes), name
    bad = torch.tensor([1.0, float("inf"), 2.0, 3.0], device=cuda)
    st, _, _, _, _ = _noalloc(bad, 1, 4, L.ROUND_RNE, 0, with_status=False)
    torch.cuda.synchronize()
    assert st == L.OK                                          # nothing to report into
