"""GPU: the ModelRunner adapter — a Llama-shaped decoder on the quantized kernels against a plain fp32 torch statement
of the same layer stack (same dequantized weights, no activation or KV quantization), and the ModelRunner contract."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dense(lin):
    return lin.codes.view(torch.float8_e4m3fn).to(torch.float32) * lin.scales[:, None]


def _reference_logits(runner, token_ids, positions, seqs_rows):
    """fp32 forward over full sequences: token_ids [tokens], positions [tokens], seqs_rows = [(r0, r1)] causal blocks."""
    cfg = runner.cfg
    nq, nkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim

    def rms(x, g):
        return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + cfg.eps) * g.to(torch.float32)

    def rope(t):
        ang = positions.to(torch.float32)[:, None] * runner.inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = t[..., : d // 2], t[..., d // 2:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)

    res = runner.embed[token_ids.long()].to(torch.float32)
    tokens = res.shape[0]
    for layer in runner.layers:
        h = rms(res, layer.g_attn)
        qkv = h @ _dense(layer.qkv).T
        q = rope(qkv[:, : nq * d].reshape(tokens, nq, d))
        k = rope(qkv[:, nq * d: (nq + nkv) * d].reshape(tokens, nkv, d))
        v = qkv[:, (nq + nkv) * d:].reshape(tokens, nkv, d)
        attn = torch.empty(tokens, nq, d, device=res.device)
        for r0, r1 in seqs_rows:
            kf = k[r0:r1].repeat_interleave(nq // nkv, dim=1)
            vf = v[r0:r1].repeat_interleave(nq // nkv, dim=1)
            s = torch.einsum("qhd,khd->hqk", q[r0:r1], kf) / math.sqrt(d)
            n = r1 - r0
            s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=res.device), 1)[None], float("-inf"))
            attn[r0:r1] = torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), vf)
        res = res + attn.reshape(tokens, nq * d) @ _dense(layer.o).T
        h = rms(res, layer.g_mlp)
        gu = h @ _dense(layer.gate_up).T
        g, u = gu[:, : cfg.ffn], gu[:, cfg.ffn:]
        res = res + (g / (1.0 + torch.exp(-g)) * u) @ _dense(layer.down).T
    return rms(res, runner.g_final) @ _dense(runner.lm_head).T


def _rel_rms(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))


def test_prefill_and_decode_against_fp32_statement(cuda):
    from oxicuda_b200.model_runner import LlamaConfig, QuantizedLlamaRunner
    cfg = LlamaConfig()
    runner = QuantizedLlamaRunner(cfg, cuda, seed=7)
    rng = np.random.default_rng(61)
    lens = [5, 23, 16]
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]
    tables = [[0, 1], [2, 3, 4], [5, 6]]                     # 16-token pages, room for the decode steps below
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    flat = [t for p in prompts for t in p]
    logits = runner.prefill(flat, starts, tables)
    assert len(logits) == 3 and len(logits[0]) == cfg.vocab_size
    ids = torch.tensor(flat, device=cuda)
    pos = torch.cat([torch.arange(n, device=cuda) for n in lens])
    ref = _reference_logits(runner, ids, pos, [(starts[i], starts[i + 1]) for i in range(3)])
    ref_last = ref[[s - 1 for s in starts[1:]]].cpu().numpy()
    # FP8 (3 mantissa bits) activations per token, FP8 weights shared with the reference, INT8 KV: a few percent
    assert _rel_rms(logits, ref_last) <= 5e-2
    # two decode steps: the cache written by prefill and by the first step is what the next step attends to
    seq_lens = list(lens)
    for step in range(2):
        nxt = [int(np.argmax(row)) for row in logits]
        logits = runner.decode(nxt, tables, seq_lens)
        for i in range(3):
            prompts[i].append(nxt[i])
        seq_lens = [n + 1 for n in seq_lens]
        flat = [t for p in prompts for t in p]
        st = [0]
        for n in seq_lens:
            st.append(st[-1] + n)
        ids = torch.tensor(flat, device=cuda)
        pos = torch.cat([torch.arange(n, device=cuda) for n in seq_lens])
        ref = _reference_logits(runner, ids, pos, [(st[i], st[i + 1]) for i in range(3)])
        assert _rel_rms(logits, ref[[s - 1 for s in st[1:]]].cpu().numpy()) <= 5e-2, step
    # a prefill of the extended prompts into fresh pages agrees with prefill + decode (same kernels, other batch shapes)
    fresh = runner.prefill(flat, st, [[10, 11], [12, 13, 14], [15, 16]])
    assert _rel_rms(fresh, logits) <= 3e-2


def test_model_runner_contract(cuda):
    from oxicuda_b200 import _lib
    from oxicuda_b200.model_runner import EmptyBatch, LlamaConfig, MockModelRunner, QuantizedLlamaRunner
    mock = MockModelRunner(8, 1)
    assert mock.vocab_size() == 8
    out = mock.decode([3, 7], [[0], [1]], [4, 9])
    assert out[0].index(10.0) == 4 and out[1].index(10.0) == 0 and sum(out[0]) == 10.0
    assert mock.prefill([1, 2, 3, 4, 5], [0, 2, 5], [[0], [1]])[1].index(10.0) == 6
    runner = QuantizedLlamaRunner(LlamaConfig(n_layers=1), cuda)
    for r in (mock, runner):
        with pytest.raises(EmptyBatch):
            r.decode([], [], [])
        with pytest.raises(_lib.DimensionMismatch):
            r.decode([1, 2], [[0]], [0, 0])
    with pytest.raises(_lib.DimensionMismatch):           # a sequence longer than its block table
        runner.decode([1], [[0]], [16])
    with pytest.raises(EmptyBatch):
        runner.prefill([], [0], [])
