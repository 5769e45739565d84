"""GPU: INT4 group-scaled weight-only linear through the C ABI — pack/unpack and the reference-order GEMM bit-exact
against the CPU oracle, the decode GEMV within 1e-2 of it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _weights(rng, N, K, group):
    vals = rng.integers(-8, 8, (N, K)).astype(np.int8)
    vals[0, :8] = [0, 1, -1, 7, -8, 3, -5, 2]
    scales = rng.uniform(0.002, 0.05, (N, K // group)).astype(np.float16)
    return vals, scales


def test_pack_unpack_reference_cases(cuda, kat, oracle):
    from oxicuda_b200 import _lib
    from oxicuda_b200.blas import Int4GemmConfig, pack_int4, unpack_int4
    k = kat["int4"]
    v = k["pack_unpack_roundtrip"]["values"]
    packed = pack_int4(torch.tensor(v, dtype=torch.int8))
    assert packed.numel() == 1 and unpack_int4(packed).tolist() == v
    with pytest.raises(_lib.InvalidArgument):
        pack_int4(torch.tensor(k["pack_wrong_length"]["values"], dtype=torch.int8))
    with pytest.raises(_lib.InvalidArgument):
        pack_int4(torch.tensor(k["pack_out_of_range"]["values"], dtype=torch.int8))
    for word, vals in k["unpack_words"]["cases"]:
        assert unpack_int4(word).tolist() == vals
    rng = np.random.default_rng(51)
    vals = rng.integers(-8, 8, 8 * 100003).astype(np.int8)
    packed = pack_int4(_t(vals, cuda))
    ref, st = oracle.pack_int4(vals)
    assert st == 0 and np.array_equal(packed.cpu().numpy().view(np.uint32), ref)
    assert np.array_equal(unpack_int4(packed).cpu().numpy(), vals)
    for m, n, kk, g in k["config_validation"]["ok"]:
        Int4GemmConfig(m, n, kk, group_size=g).validate()
    for m, n, kk, g in k["config_validation"]["bad"]:
        with pytest.raises((_lib.InvalidDimension, _lib.InvalidArgument)):
            Int4GemmConfig(m, n, kk, group_size=g).validate()
    kk, g, want = k["helpers"]["num_groups"]
    assert Int4GemmConfig(128, 128, kk, group_size=g).num_groups() == want
    assert Int4GemmConfig(128, 128, k["helpers"]["packed_k"][0]).packed_k() == k["helpers"]["packed_k"][1]
    m, n, kk, la, lb, g = k["kernel_name"]["config"]
    name = Int4GemmConfig(m, n, kk, la, lb, g).kernel_name()
    assert all(part in name for part in k["kernel_name"]["contains"])
    assert list(Int4GemmConfig(1, 1, 8).tile_config()) == k["tile_config_sm100"]["tile"]


def test_gemm_int4_reference_order_bit_exact(cuda, oracle):
    from oxicuda_b200 import _lib
    from oxicuda_b200._lib import default_handle, ptr
    from oxicuda_b200.blas import Int4GemmConfig, gemm_int4
    rng = np.random.default_rng(52)
    for M, N, K, group in ((1, 1, 8, 8), (5, 3, 64, 32), (33, 7, 256, 64), (128, 40, 1024, 128), (257, 1, 4096, 256), (64, 65, 48, 16)):
        vals, scales = _weights(rng, M, K, group)
        packed, _ = oracle.pack_int4(vals)
        b = rng.standard_normal((K, N)).astype(np.float32)
        ref = oracle.gemm_int4(packed, scales, b, M, N, K, group)
        got = gemm_int4(_t(packed.view(np.int32), cuda), _t(scales, cuda), _t(b, cuda), Int4GemmConfig(M, N, K, group_size=group))
        assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32)), (M, N, K, group)
    h = default_handle()
    z = torch.zeros(64, dtype=torch.int32, device=cuda)
    for bad, err in (((4, 4, 100, 32), _lib.InvalidDimension), ((4, 0, 64, 32), _lib.InvalidDimension), ((4, 4, 64, 3), _lib.InvalidArgument),
                     ((4, 4, 48, 32), _lib.InvalidArgument)):
        with pytest.raises(err):
            h.call("b2q_gemm_int4_f32", ptr(z), ptr(z), ptr(z), ptr(z), *bad)


@pytest.mark.parametrize("group", [32, 64, 128, 256])
def test_gemv_int4_decode(cuda, oracle, group):
    from oxicuda_b200 import _lib
    from oxicuda_b200.blas import gemv_int4_wo
    rng = np.random.default_rng(53 + group)
    for tokens, N, K in ((1, 64, 512), (3, 100, 1024), (8, 4096, 4096), (16, 1000, 2048), (32, 300, 1536), (5, 16, 256), (1, 14336, 4096)):
        vals, scales = _weights(rng, N, K, group)
        packed, _ = oracle.pack_int4(vals)
        x = torch.from_numpy(rng.standard_normal((tokens, K)).astype(np.float32)).to(torch.bfloat16)
        ref = oracle.gemm_int4(packed, scales, x.float().numpy().T.copy(), N, tokens, K, group).T      # [tokens, N]
        got = gemv_int4_wo(_t(packed.view(np.int32), cuda), _t(scales, cuda), group, x.to(cuda), N, K, out_dtype=torch.float32)
        got = got.cpu().numpy()
        tau = 1e-3 * np.sqrt((ref.astype(np.float64) ** 2).mean())
        err = (np.abs(got - ref) / np.maximum(np.abs(ref), tau)).max()
        assert err <= 1e-2, (tokens, N, K, group, err)
        out16 = gemv_int4_wo(_t(packed.view(np.int32), cuda), _t(scales, cuda), group, x.to(cuda), N, K)
        assert torch.equal(out16.cpu(), torch.from_numpy(got).to(torch.bfloat16)), (tokens, N, K, group)
    p = torch.zeros(64 * 24, dtype=torch.int32, device=cuda)
    s = torch.zeros(64 * 6, dtype=torch.float16, device=cuda)
    with pytest.raises(_lib.UnsupportedOperation):       # K % 128 != 0 belongs to the reference-order entry point
        gemv_int4_wo(p, s, 32, torch.zeros(1, 192, dtype=torch.bfloat16, device=cuda), 64, 192)
    with pytest.raises(_lib.UnsupportedOperation):
        gemv_int4_wo(p, s, 32, torch.zeros(33, 128, dtype=torch.bfloat16, device=cuda), 64, 128)
