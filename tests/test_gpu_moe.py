"""GPU: FP8 mixture-of-experts layer (top-k routing, token scatter, grouped gate|up and down GEMMs, SwiGLU +
re-quantize, weighted gather) against the oracle composition of the reference's router, dispatcher and SwiGLU
expert on the same seeded inputs.  Tolerance as for the MLP: |got - ref| <= 1e-2*|ref| + 1e-2*rms(ref)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


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
        gu = oracle.gemm_fp8(xc.reshape(-1, hidden), wc.reshape(2 * F, hidden), xs, ws, 0, 1, "bf16")
        hh = oracle.swiglu(gu[:, :F], gu[:, F:])
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
