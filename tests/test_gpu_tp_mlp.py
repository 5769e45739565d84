"""GPU: tensor-parallel FP8 SwiGLU MLP (gate/up column-parallel, down row-parallel + all-reduce) against the
oracle composition on the same seeded inputs.  tp=1 runs in-process; tp=2 runs as two NCCL ranks when the box
has two GPUs.  Tolerance: |got - ref| <= 1e-2*|ref| + 1e-2*rms(ref) on every element (1e-2 relative, as for the
GEMMs, plus an absolute floor): exp() may differ in the last bit between libm and the GPU, which can move one
re-quantized SwiGLU value to the neighbouring E4M3 code; when that value is the row's largest, one output
moves by up to about 7e-3*rms."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def oracle_mlp(oracle, x_bf16_as_f32, wg, wu, wd, tp):
    """Reference composition, ranks simulated in order (crates/oxicuda-dist-infer/src/lib.rs:154-183)."""
    tokens, hidden = x_bf16_as_f32.shape
    ffn = wg.shape[0]
    F = ffn // tp
    xc, xs, _ = oracle.fp8_quantize_rows(x_bf16_as_f32, tokens, hidden, 0, 1)
    xc = xc.reshape(tokens, hidden)
    total = None
    for r in range(tp):
        wgu = np.concatenate([wg[r * F:(r + 1) * F], wu[r * F:(r + 1) * F]], axis=0)
        wc, ws, _ = oracle.fp8_quantize_rows(wgu, 2 * F, hidden, 0, 1)
        inter = F % 128 == 0 and hidden % 16 == 0            # TpFp8Mlp then holds the gate | up shard interleaved per 128 rows
        if inter:
            wc, ws = oracle.interleave_rows128(wc.reshape(2 * F, hidden)[:F], wc.reshape(2 * F, hidden)[F:]), oracle.interleave_rows128(ws[:F], ws[F:])
        h = oracle.swiglu_mlp_hidden(xc, xs, wc, ws, tokens, hidden, F, inter)
        hc, hs, _ = oracle.fp8_quantize_rows(h, tokens, F, 0, 1)
        wdc, wds, _ = oracle.fp8_quantize_rows(np.ascontiguousarray(wd[:, r * F:(r + 1) * F]), hidden, F, 0, 1)
        part = _bf16_round(oracle.gemm_fp8(hc.reshape(tokens, F), wdc.reshape(hidden, F), hs, wds, 0, 1, "f32"))
        total = part if total is None else _bf16_round(total + part)
    return total


def rel_err(got, ref):
    """max over elements of |got - ref| / (|ref| + rms(ref)); <= 1e-2 means the bound of the module docstring."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    rms = np.sqrt((ref ** 2).mean()) + 1e-30
    return float((np.abs(got - ref) / (np.abs(ref) + rms)).max())


def make_inputs(tokens, hidden, ffn, seed=0xB2000003):
    rng = np.random.default_rng(seed)
    x = _bf16_round(rng.standard_normal((tokens, hidden)))
    wg = (rng.standard_normal((ffn, hidden)) * 0.01).astype(np.float32)
    wu = (rng.standard_normal((ffn, hidden)) * 0.01).astype(np.float32)
    wd = (rng.standard_normal((hidden, ffn)) * 0.01).astype(np.float32)
    return x, wg, wu, wd


@pytest.mark.parametrize("tokens", [1, 64, 300])
def test_mlp_tp1_matches_oracle(cuda, oracle, tokens):
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp
    hidden, ffn = 512, 1536
    x, wg, wu, wd = make_inputs(tokens, hidden, ffn)
    t = lambda a: torch.from_numpy(a).to(cuda)
    mlp = TpFp8Mlp(t(wg), t(wu), t(wd), DistInferHandle(0, ParallelismConfig(tp=1)))
    y = mlp.forward(t(x).to(torch.bfloat16)).float().cpu().numpy()
    ref = oracle_mlp(oracle, x, wg, wu, wd, 1)
    assert rel_err(y, ref) <= 1e-2
    # median relative error is at the bf16 rounding level
    assert np.median(np.abs(y - ref) / (np.abs(ref) + 1e-6)) < 5e-3


@pytest.mark.parametrize("tokens", [1, 64])
def test_mlp_at_stated_size_hidden8192_ffn28672(cuda, oracle, tokens):
    """The tensor-parallel MLP configuration at its stated size (hidden 8192, FFN 28672; 1 and 64 tokens): the un-sharded
    layer through b2q_mlp_swiglu_fp8_forward, and the layer cut into 8 tensor-parallel shards run on this one GPU
    (every shard's partial, added in rank order), each against the oracle composition over the same codes."""
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp
    hidden, ffn = 8192, 28672
    g = torch.Generator(device=cuda).manual_seed(0xB2000003)
    wg = torch.randn(ffn, hidden, device=cuda, generator=g) * 0.01
    wu = torch.randn(ffn, hidden, device=cuda, generator=g) * 0.01
    wd = torch.randn(hidden, ffn, device=cuda, generator=g) * 0.01
    x = torch.randn(tokens, hidden, device=cuda, generator=g).to(torch.bfloat16)
    xf = x.float().cpu().numpy()
    xc, xs, _ = oracle.fp8_quantize_rows(xf, tokens, hidden, 0, 1)

    def oracle_over(shards):
        total = None
        for sh in shards:
            F = sh.local_ffn
            inter = sh.gu_codes is not None
            h = oracle.swiglu_mlp_hidden(xc, xs, (sh.gu_codes if inter else sh.gate_up.codes).cpu().numpy(),
                                         (sh.gu_scales if inter else sh.gate_up.scales).cpu().numpy(), tokens, hidden, F, inter)
            hc, hs, _ = oracle.fp8_quantize_rows(h, tokens, F, 0, 1)
            part = _bf16_round(oracle.gemm_fp8(hc.reshape(tokens, F), sh.down.codes.cpu().numpy(), hs, sh.down.scales.cpu().numpy(), 0, 1, "f32"))
            total = part if total is None else _bf16_round(total + part)
        return total

    full = TpFp8Mlp(wg, wu, wd, DistInferHandle(0, ParallelismConfig(tp=1)))
    y = full.forward(x).float().cpu().numpy()
    assert rel_err(y, oracle_over([full])) <= 1e-2
    del full
    shards = [TpFp8Mlp(wg, wu, wd, DistInferHandle(r, ParallelismConfig(tp=8))) for r in range(8)]
    del wg, wu, wd
    total = None
    for sh in shards:                                       # what the 8 ranks compute, one after the other on this GPU
        part = sh.forward_partial(x).float()
        total = part if total is None else (total + part).to(torch.bfloat16).float()
    # eight independent re-quantizations of the SwiGLU result (one per shard) give eight chances for an exp() last-bit
    # difference to move a row's largest value to the neighbouring E4M3 code: twice the single-layer bound
    assert rel_err(total.cpu().numpy(), oracle_over(shards)) <= 2e-2


def test_swiglu_quantize_kernel_against_oracle(cuda, oracle):
    from oxicuda_b200 import _lib as L
    rng = np.random.default_rng(9)
    rows, cols = 37, 1000                       # ragged: scalar path; and a vectorised case below
    for rows, cols in ((37, 1000), (64, 2048)):
        gu = torch.from_numpy(rng.standard_normal((rows, 2 * cols)).astype(np.float32) * 3).to(torch.bfloat16).to(cuda)
        codes = torch.empty(rows, cols, dtype=torch.uint8, device=cuda)
        scales = torch.empty(rows, dtype=torch.float32, device=cuda)
        L.default_handle().call("b2q_swiglu_quantize_rows_bf16", L.ptr(gu), L.ptr(gu[:, cols:]), rows, cols, 2 * cols,
                                L.FP8_E4M3, L.ROUND_RNE, L.ptr(scales), L.ptr(codes))
        guf = gu.float().cpu().numpy()
        h = oracle.swiglu(guf[:, :cols], guf[:, cols:])
        c_ref, s_ref, _ = oracle.fp8_quantize_rows(h, rows, cols, 0, 1)
        assert np.allclose(scales.cpu().numpy(), s_ref, rtol=1e-6)
        dec_got = oracle.fp8_decode(codes.cpu().numpy().reshape(-1), 0, 1)
        dec_ref = oracle.fp8_decode(c_ref, 0, 1)
        mism = np.count_nonzero(codes.cpu().numpy().reshape(-1) != c_ref)
        assert mism <= 1e-3 * c_ref.size, mism           # exp() last-bit differences may flip a code on a boundary
        assert np.abs(dec_got - dec_ref).max() <= 32.0   # and then only to the neighbouring code (<= one E4M3 step)


def test_mlp_tp2_two_ranks(cuda, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "tp_mlp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "TP2 OK" in r.stdout
