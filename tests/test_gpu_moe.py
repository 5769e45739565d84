"""GPU: FP8 mixture-of-experts layer (top-k routing, token scatter, grouped gate|up and down GEMMs, SwiGLU +
re-quantize, weighted gather) against the oracle composition of the reference's router, dispatcher and SwiGLU
expert on the same seeded inputs.  Tolerance as for the MLP: |got - ref| <= 1e-2*|ref| + 1e-2*rms(ref)."""
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


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def oracle_route(logits, top_k):
    """TopKRouter::route (crates/oxicuda-dist-infer/src/expert_parallel/router.rs:94-140)."""
    order = np.argsort(-logits, axis=1, kind="stable")[:, :top_k]
    top = np.take_along_axis(logits, order, axis=1)
    e = np.exp((top - top[:, :1]).astype(np.float32))
    w = e / e.sum(axis=1, keepdims=True)
    return order, w.astype(np.float32)


def oracle_moe(oracle, x, logits, experts, top_k):
    tokens, hidden = x.shape
    idx, wgt = oracle_route(logits, top_k)
    ys = {}
    for e, (w1, w3, w2) in enumerate(experts):
        toks = np.nonzero((idx == e).any(axis=1))[0]
        if toks.size == 0:
            continue
        F = w1.shape[0]
        xe = x[toks]
        xc, xs, _ = oracle.fp8_quantize_rows(xe, toks.size, hidden, 0, 1)
        wc, ws, _ = oracle.fp8_quantize_rows(np.concatenate([w1, w3], 0), 2 * F, hidden, 0, 1)
        inter = F % 128 == 0 and hidden % 16 == 0            # MoeFp8Layer then holds every expert's gate | up rows interleaved per 128
        if inter:
            wc, ws = oracle.interleave_rows128(wc.reshape(2 * F, hidden)[:F], wc.reshape(2 * F, hidden)[F:]), oracle.interleave_rows128(ws[:F], ws[F:])
        hh = oracle.swiglu_mlp_hidden(xc, xs, wc, ws, toks.size, hidden, F, inter)
        hc, hs, _ = oracle.fp8_quantize_rows(hh, toks.size, F, 0, 1)
        w2c, w2s, _ = oracle.fp8_quantize_rows(w2, hidden, F, 0, 1)
        y = oracle.gemm_fp8(hc.reshape(-1, F), w2c.reshape(hidden, F), hs, w2s, 0, 1, "bf16")
        for i, t in enumerate(toks):
            ys[(int(t), e)] = y[i]
    out = np.zeros((tokens, hidden), np.float32)
    for t in range(tokens):
        acc = np.zeros(hidden, np.float32)
        for j in range(top_k):                       # gather: sum of weight * expert_out in plan order
            acc = acc + wgt[t, j] * ys[(t, int(idx[t, j]))]
        out[t] = acc
    return _bf16(out), idx, wgt


def err(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    rms = np.sqrt((ref ** 2).mean()) + 1e-30
    return float((np.abs(got - ref) / (np.abs(ref) + rms)).max())


@pytest.mark.parametrize("tokens,n_experts,top_k", [(96, 4, 2), (5, 8, 2), (200, 8, 1)])
def test_moe_layer_matches_oracle(cuda, oracle, tokens, n_experts, top_k):
    from oxicuda_b200.dist_infer import DistInferHandle, MoeFp8Layer, ParallelismConfig, TopKRouter
    rng = np.random.default_rng(0xB2000004 + tokens)
    hidden, ffn = 256, 512
    x = _bf16(rng.standard_normal((tokens, hidden)))
    logits = rng.standard_normal((tokens, n_experts)).astype(np.float32)
    if n_experts == 8 and tokens == 200:
        logits[:, 3] = -50.0                          # an expert that receives no token
    experts = [((rng.standard_normal((ffn, hidden)) * 0.02).astype(np.float32),
                (rng.standard_normal((ffn, hidden)) * 0.02).astype(np.float32),
                (rng.standard_normal((hidden, ffn)) * 0.02).astype(np.float32)) for _ in range(n_experts)]
    ref, idx, wgt = oracle_moe(oracle, x, logits, experts, top_k)
    t = lambda a: torch.from_numpy(a).to(cuda)
    plan = TopKRouter(n_experts, top_k).route(t(logits), tokens)
    assert np.array_equal(plan.expert_idx.cpu().numpy(), idx.astype(np.int32))
    assert np.allclose(plan.weight.cpu().numpy(), wgt, rtol=1e-6, atol=1e-7)
    assert int(plan.expert_load.sum()) == tokens * top_k
    layer = MoeFp8Layer([(t(a), t(b), t(c)) for a, b, c in experts], n_experts, top_k,
                        DistInferHandle(0, ParallelismConfig(ep=1)))
    y = layer.forward(t(x).to(torch.bfloat16), t(logits)).float().cpu().numpy()
    assert err(y, ref) <= 1e-2


def test_scatter_gather_identity(cuda):
    """e2e_ep_moe_dispatch_gather of the reference (crates/oxicuda-dist-infer/src/lib.rs:231-273): identity experts
    and weights that sum to one give the input back."""
    from oxicuda_b200 import _lib as L
    tokens, hidden, k = 50, 128, 2
    x = torch.randn(tokens, hidden, device=cuda).to(torch.bfloat16)
    tok = torch.arange(tokens, device=cuda, dtype=torch.int32).repeat_interleave(k)
    perm = torch.randperm(tokens * k, device=cuda).to(torch.int32)
    buf = torch.empty(tokens * k, hidden, dtype=torch.bfloat16, device=cuda)
    h = L.default_handle()
    h.call("b2q_ep_token_scatter", L.ptr(x), L.ptr(tok), L.ptr(perm), tokens * k, hidden * 2, L.ptr(buf))
    w = torch.full((tokens * k,), 0.5, device=cuda)
    out = torch.empty_like(x)
    h.call("b2q_ep_token_gather_bf16", L.ptr(buf), L.ptr(perm), L.ptr(w), tokens, k, hidden, L.ptr(out))
    assert torch.equal(out, x)


def test_grouped_gemm_rows_device_table(cuda, oracle):
    """b2q_grouped_gemm_fp8_rows: one launch over a device-side table of problems with different row counts (an empty one,
    a tiny one, one that is exactly a tile, a ragged one) against the oracle's GEMM per problem."""
    from oxicuda_b200 import _lib as L
    from oxicuda_b200.quant import Fp8Codec
    rng = np.random.default_rng(12)
    N, K = 384, 512
    counts = [300, 0, 17, 256, 1000]
    offs, o = [], 0
    for c in counts:
        offs.append(o)
        o += (c + 255) // 256 * 256
    offs.append(o)
    cap = o
    G = len(counts)
    codec = Fp8Codec.e4m3("rne")
    a = torch.zeros(cap, K, device=cuda)
    for g, c in enumerate(counts):
        a[offs[g]:offs[g] + c] = torch.from_numpy(rng.standard_normal((c, K)).astype(np.float32)).to(cuda)
    w = torch.from_numpy((rng.standard_normal((G * N, K)) * 0.05).astype(np.float32)).to(cuda)
    ac, sa = codec.quantize_rows(a, cap, K)
    wc, sw = codec.quantize_rows(w, G * N, K)
    out = torch.zeros(cap, N, dtype=torch.float32, device=cuda)
    cnt_d = torch.tensor(counts, dtype=torch.int32, device=cuda)
    off_d = torch.tensor(offs, dtype=torch.int32, device=cuda)
    L.default_handle().call("b2q_grouped_gemm_fp8_rows", L.ptr(ac), L.ptr(sa), L.ptr(wc), L.ptr(sw), L.ptr(off_d), L.ptr(cnt_d), G, cap, N, K,
                            L.FP8_E4M3, L.ptr(out), L.OUT_F32)
    L.default_handle().check()
    acn, wcn = ac.view(cap, K).cpu().numpy(), wc.view(G * N, K).cpu().numpy()
    san, swn = sa.cpu().numpy(), sw.cpu().numpy()
    got = out.cpu().numpy()
    for g, c in enumerate(counts):
        if c == 0:
            continue
        rows = slice(offs[g], offs[g] + c)
        ref = np.asarray(oracle.gemm_fp8(acn[rows], wcn[g * N:(g + 1) * N], san[rows], swn[g * N:(g + 1) * N], 0, 1, "f32")).reshape(c, N)
        assert err(got[rows], ref) <= 1e-3, g
    # rows of the padding after the empty and the tiny problem were never touched by another problem's tile
    assert not np.any(got[offs[2] + 256:offs[3]]) if offs[3] - offs[2] > 256 else True


def test_mixtral_shaped_moe_at_stated_size(cuda, oracle):
    """The grouped-MoE configuration at its stated size: 8 experts of 4096 -> 14336 -> 4096, top-2 routing over 4096 tokens
    with per-expert counts drawn from a seeded Dirichlet(1) multinomial; the whole layer runs on the GPU in one call, the
    oracle composition (over the layer's own codes) checks a 96-token subset."""
    from oxicuda_b200.dist_infer import DistInferHandle, MoeFp8Layer, ParallelismConfig
    E, hidden, ffn, tokens, top_k = 8, 4096, 14336, 4096, 2
    rng = np.random.default_rng(0xB2000005)
    prob = rng.dirichlet(np.ones(E))
    logits = np.full((tokens, E), -30.0, np.float32)
    for t in range(tokens):
        pair = rng.choice(E, size=2, replace=False, p=prob)         # two distinct experts, drawn in proportion to p
        logits[t, pair] = 20.0 + rng.standard_normal(2).astype(np.float32)   # gate weights: softmax of two N(0,1) logits
    g = torch.Generator(device=cuda).manual_seed(0xB2000005)
    experts = []
    for _ in range(E):
        experts.append((torch.randn(ffn, hidden, device=cuda, generator=g) * 0.02, torch.randn(ffn, hidden, device=cuda, generator=g) * 0.02,
                        torch.randn(hidden, ffn, device=cuda, generator=g) * 0.02))
    layer = MoeFp8Layer(experts, E, top_k, DistInferHandle(0, ParallelismConfig(ep=1)))
    del experts
    torch.cuda.empty_cache()
    x = torch.randn(tokens, hidden, device=cuda, generator=g).to(torch.bfloat16)
    y = layer.forward(x, torch.from_numpy(logits).to(cuda))
    from oxicuda_b200._lib import default_handle
    default_handle().check()
    counts = layer.last_counts.cpu().numpy()
    idx, wgt = oracle_route(logits, top_k)
    assert counts.sum() == tokens * top_k
    assert np.array_equal(counts, np.bincount(idx.reshape(-1), minlength=E))
    # oracle on a subset of tokens, expert by expert, over the layer's own codes and scales
    sub = np.arange(0, tokens, tokens // 96)[:96]
    xs_f = x[torch.from_numpy(sub).to(cuda)].float().cpu().numpy()
    ref = np.zeros((sub.size, hidden), np.float32)
    parts = {}
    F = ffn
    for e in range(E):
        rows = [i for i, t in enumerate(sub) if e in idx[t]]
        if not rows:
            continue
        xe = xs_f[rows]
        xc, xsc, _ = oracle.fp8_quantize_rows(xe, len(rows), hidden, 0, 1)
        hh = oracle.swiglu_mlp_hidden(xc, xsc, layer.gate_up_codes[e].cpu().numpy(), layer.gate_up_scales[e * 2 * F:(e + 1) * 2 * F].cpu().numpy(),
                                      len(rows), hidden, F, layer.interleaved)
        hc, hs, _ = oracle.fp8_quantize_rows(hh, len(rows), F, 0, 1)
        ye = oracle.gemm_fp8(hc.reshape(-1, F), layer.down_codes[e].cpu().numpy(), hs, layer.down_scales[e * hidden:(e + 1) * hidden].cpu().numpy(),
                             0, 1, "bf16")
        for k, i in enumerate(rows):
            parts[(i, e)] = ye[k]
    for i, t in enumerate(sub):
        acc = np.zeros(hidden, np.float32)
        for j in range(top_k):
            acc = acc + wgt[t, j] * parts[(i, int(idx[t, j]))]
        ref[i] = acc
    got = y[torch.from_numpy(sub).to(cuda)].float().cpu().numpy()
    assert err(got, _bf16(ref)) <= 1e-2


def test_moe_expert_parallel_two_ranks(cuda, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "moe_ep_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "EP2 OK" in r.stdout


def _mx_e4m3(oracle, x):
    """One E4M3 code per value under a power-of-two scale per 32 values (smallest 2^e with max / 2^e <= 448): the
    activation quantizer of the block-scaled FP4 GEMM in its W4A8 mode; returns the dequantized values (exact in bf16)."""
    rows, K = x.shape
    xf = np.asarray(x, np.float32).reshape(rows, K // 32, 32)
    amax = np.abs(xf).max(axis=2, keepdims=True)
    e = np.where(amax > 0, np.ceil(np.log2(np.maximum(amax, 1e-38) / 448.0)), 0.0)
    e = np.maximum(e, -127.0)
    q = oracle.fp8_decode(oracle.fp8_encode((xf / np.exp2(e)).astype(np.float32).reshape(-1), 0, 1)[0], 0, 1).reshape(xf.shape) * np.exp2(e)
    return q.reshape(rows, K).astype(np.float32)


def _bits(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("tokens,n_experts,top_k", [(200, 4, 2), (700, 8, 2)])
def test_moe_fp4_layer_matches_oracle(cuda, oracle, tokens, n_experts, top_k):
    """b2q_moe_forward_fp4 / b2q_grouped_gemm_fp4_rows: block-scaled FP4 experts, both grouped GEMMs one launch each of the
    tcgen05 block-scaled kernel over a device-side table.  Oracle: the router and the gather of the reference, and per expert
    the activation quantizer above, dequantize_fp4 + f32 dot (the oracle's FP4 product), silu(gate) * up in f32, bf16
    where the layer stores bf16; over the layer's own codes."""
    from oxicuda_b200.dist_infer import DistInferHandle, MoeFp4Layer, ParallelismConfig
    rng = np.random.default_rng(0xB2000006 + tokens)
    hidden, ffn = 256, 384
    x = _bf16(rng.standard_normal((tokens, hidden)))
    logits = rng.standard_normal((tokens, n_experts)).astype(np.float32)
    if n_experts == 8:
        logits[:, 5] = -50.0                                        # an expert that receives no token
    experts = [((rng.standard_normal((ffn, hidden)) * 0.05).astype(np.float32), (rng.standard_normal((ffn, hidden)) * 0.05).astype(np.float32),
                (rng.standard_normal((hidden, ffn)) * 0.05).astype(np.float32)) for _ in range(n_experts)]
    t = lambda a: torch.from_numpy(a).to(cuda)
    layer = MoeFp4Layer([(t(a), t(b), t(c)) for a, b, c in experts], n_experts, top_k, DistInferHandle(0, ParallelismConfig(ep=1)))
    y = layer.forward(t(x).to(torch.bfloat16), t(logits)).float().cpu().numpy()
    from oxicuda_b200._lib import default_handle
    default_handle().check()
    idx, wgt = oracle_route(logits, top_k)
    counts = np.bincount(idx.reshape(-1), minlength=n_experts)
    assert np.array_equal(layer.last_counts.cpu().numpy(), counts.astype(np.int32))
    F = ffn
    gc = layer.gate_up_codes.cpu().numpy().reshape(n_experts, 2 * F * hidden // 2)
    gs = layer.gate_up_scales.cpu().numpy().reshape(n_experts, 2 * F * hidden // 32)
    dc = layer.down_codes.cpu().numpy().reshape(n_experts, hidden * F // 2)
    ds = layer.down_scales.cpu().numpy().reshape(n_experts, hidden * F // 32)
    ys = {}
    for e in range(n_experts):
        toks = np.nonzero((idx == e).any(axis=1))[0]
        if toks.size == 0:
            continue
        xq = _mx_e4m3(oracle, x[toks])
        gu = _bf16(np.asarray(oracle.gemv_fp4(gc[e], gs[e], _bits(xq), toks.size, 2 * F, hidden, 32, "f32")).reshape(toks.size, 2 * F))
        h = _bf16(oracle.swiglu(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:])))
        ye = _bf16(np.asarray(oracle.gemv_fp4(dc[e], ds[e], _bits(_mx_e4m3(oracle, h)), toks.size, hidden, F, 32, "f32")).reshape(toks.size, hidden))
        for i, tk in enumerate(toks):
            ys[(int(tk), e)] = ye[i]
    ref = np.zeros((tokens, hidden), np.float32)
    for tk in range(tokens):
        acc = np.zeros(hidden, np.float32)
        for j in range(top_k):
            acc = acc + wgt[tk, j] * ys[(tk, int(idx[tk, j]))]
        ref[tk] = acc
    assert err(y, _bf16(ref)) <= 1e-2
