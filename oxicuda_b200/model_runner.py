"""The caller of the quantized linear path: a `ModelRunner` (crates/oxicuda-infer/src/executor/model_runner.rs:24-64)
over a Llama-shaped decoder whose linears, norm+quantize steps and KV cache run on the kernels of this library.

Per layer and step: `rms_norm_quantize_fp8` (residual add + RMSNorm + per-token FP8) -> fused q|k|v FP8 GEMM -> rotary
embedding -> per-token INT8 KV-cache quantization into a paged cache (`b2q_kv_quantize_tokens_bf16`, the scheme of
crates/oxicuda-infer/src/cache/kv_quant.rs) -> attention over the dequantized pages -> per-token FP8 -> o projection ->
`rms_norm_quantize_fp8` -> gate|up FP8 GEMM -> `b2q_swiglu_quantize_rows_bf16` -> down FP8 GEMM; the logits come from an
FP8 lm_head.  Attention itself is outside the quantized-linear path and is plain torch (softmax(QK^T/sqrt(d))V per
sequence); everything with a `b2q_` entry point goes through the C ABI.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib as L
from ._lib import default_handle, ptr
from .dist_infer import Fp8Linear
from .kv_cache import rms_norm_quantize_fp8
from .quant import Fp8Codec


class EmptyBatch(L.B2qError):
    """InferError::EmptyBatch"""


def _check_batch(n_tokens: int, *others: int):
    """The argument checks of MockModelRunner::decode (model_runner.rs:105-116)."""
    if n_tokens == 0:
        raise EmptyBatch(L.ERR_EMPTY_INPUT, "empty batch")
    for o in others:
        if o != n_tokens:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n_tokens}, got {o}")


class MockModelRunner:
    """model_runner.rs:68-150: logits 10.0 at (token + bias) % vocab_size, 0 elsewhere."""

    def __init__(self, vocab_size: int, bias: int):
        self._vocab, self.bias = vocab_size, bias

    def vocab_size(self) -> int:
        return self._vocab

    def _logits(self, token: int):
        row = [0.0] * self._vocab
        row[(token + self.bias) % self._vocab] = 10.0
        return row

    def decode(self, token_ids, block_tables, seq_lens):
        _check_batch(len(token_ids), len(block_tables), len(seq_lens))
        return [self._logits(t) for t in token_ids]

    def prefill(self, token_ids, seq_starts, block_tables):
        if len(seq_starts) < 2:
            raise EmptyBatch(L.ERR_EMPTY_INPUT, "empty batch")
        return [self._logits(token_ids[seq_starts[i + 1] - 1]) for i in range(len(seq_starts) - 1)]


@dataclass
class LlamaConfig:
    vocab_size: int = 512
    hidden: int = 256
    n_layers: int = 2
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 512
    block_size: int = 16          # tokens per KV page
    num_blocks: int = 64          # pages in the cache
    rope_theta: float = 10000.0
    eps: float = 1e-5
    kv_bits: int = 8


class _Layer:
    def __init__(self, cfg: LlamaConfig, gen, dev):
        def w(rows, cols):
            return torch.randn(rows, cols, device=dev, generator=gen) * (1.0 / math.sqrt(cols))
        qkv_rows = (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim
        self.qkv = Fp8Linear(w(qkv_rows, cfg.hidden))
        self.o = Fp8Linear(w(cfg.hidden, cfg.n_heads * cfg.head_dim))
        self.gate_up = Fp8Linear(w(2 * cfg.ffn, cfg.hidden))
        self.down = Fp8Linear(w(cfg.hidden, cfg.ffn))
        self.g_attn = (1.0 + 0.05 * torch.randn(cfg.hidden, device=dev, generator=gen)).to(torch.bfloat16)
        self.g_mlp = (1.0 + 0.05 * torch.randn(cfg.hidden, device=dev, generator=gen)).to(torch.bfloat16)
        pages = cfg.num_blocks * cfg.block_size
        # paged KV cache: codes per (page slot, kv head, channel), one (scale, zero point) per (page slot, kv head)
        self.k_codes = torch.zeros(pages, cfg.n_kv_heads, cfg.head_dim, dtype=torch.uint8, device=dev)
        self.v_codes = torch.zeros_like(self.k_codes)
        self.k_par = torch.zeros(2, pages, cfg.n_kv_heads, dtype=torch.float32, device=dev)   # [scale | zero point]
        self.v_par = torch.zeros_like(self.k_par)


class QuantizedLlamaRunner:
    """ModelRunner over random-init weights of the given shape (there are no checkpoints to load here)."""

    def __init__(self, cfg: LlamaConfig, device, seed: int = 0):
        self.cfg, self.dev = cfg, device
        gen = torch.Generator(device=device).manual_seed(seed)
        self.embed = (torch.randn(cfg.vocab_size, cfg.hidden, device=device, generator=gen) * 0.5).to(torch.bfloat16)
        self.layers = [_Layer(cfg, gen, device) for _ in range(cfg.n_layers)]
        self.g_final = (1.0 + 0.05 * torch.randn(cfg.hidden, device=device, generator=gen)).to(torch.bfloat16)
        self.lm_head = Fp8Linear(torch.randn(cfg.vocab_size, cfg.hidden, device=device, generator=gen) * (1.0 / math.sqrt(cfg.hidden)))
        self.codec = Fp8Codec.e4m3("rne")
        self.trace = None          # a list here collects every stage's tensors per layer (tests check each stage on its own inputs)
        half = cfg.head_dim // 2
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))

    def vocab_size(self) -> int:
        return self.cfg.vocab_size

    # ---- pieces -------------------------------------------------------------------------------------------------
    def _rope(self, t: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """t [tokens, heads, head_dim] bf16, rotate-half form, computed in f32."""
        ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]          # [tokens, half]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x = t.to(torch.float32)
        a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1).to(torch.bfloat16)

    def _kv_store(self, codes_buf, par_buf, kv: torch.Tensor, slots: torch.Tensor):
        """Quantizes kv [tokens, kv_heads, head_dim] bf16 per (token, head) and writes it to the page slots."""
        cfg = self.cfg
        tokens = kv.shape[0]
        rows = tokens * cfg.n_kv_heads
        kvc = kv.contiguous()
        codes = torch.empty(rows, cfg.head_dim, dtype=torch.uint8, device=self.dev)
        sc = torch.empty(rows, dtype=torch.float32, device=self.dev)
        zp = torch.empty(rows, dtype=torch.float32, device=self.dev)
        default_handle().call("b2q_kv_quantize_tokens_bf16", ptr(kvc), rows, cfg.head_dim, cfg.kv_bits, 0, ptr(codes), ptr(sc), ptr(zp))
        codes_buf[slots] = codes.view(tokens, cfg.n_kv_heads, cfg.head_dim)
        par_buf[0, slots] = sc.view(tokens, cfg.n_kv_heads)
        par_buf[1, slots] = zp.view(tokens, cfg.n_kv_heads)

    def _kv_load(self, codes_buf, par_buf, slots: torch.Tensor) -> torch.Tensor:
        """Dequantizes the page slots of one sequence -> bf16 [len, kv_heads, head_dim]."""
        cfg = self.cfg
        n = slots.numel()
        rows = n * cfg.n_kv_heads
        codes = codes_buf[slots].contiguous()
        sc = par_buf[0, slots].contiguous()
        zp = par_buf[1, slots].contiguous()
        out = torch.empty(rows, cfg.head_dim, dtype=torch.bfloat16, device=self.dev)
        default_handle().call("b2q_kv_dequantize_tokens_bf16", ptr(codes), rows, cfg.head_dim, 0, ptr(sc), ptr(zp), ptr(out))
        return out.view(n, cfg.n_kv_heads, cfg.head_dim)

    def _slots(self, table, start: int, end: int) -> torch.Tensor:
        bs = self.cfg.block_size
        if (end + bs - 1) // bs > len(table):
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {(end + bs - 1) // bs} KV blocks, got {len(table)}")
        pos = torch.arange(start, end, device=self.dev)
        blocks = torch.tensor(list(table), device=self.dev, dtype=torch.long)
        return blocks[pos // bs] * bs + pos % bs

    def _attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_start: int) -> torch.Tensor:
        """q [nq, heads, d], k / v [len, kv_heads, d]; query i sees keys 0..q_start+i.  f32 softmax."""
        cfg = self.cfg
        rep = cfg.n_heads // cfg.n_kv_heads
        kf = k.to(torch.float32).repeat_interleave(rep, dim=1)
        vf = v.to(torch.float32).repeat_interleave(rep, dim=1)
        s = torch.einsum("qhd,khd->hqk", q.to(torch.float32), kf) / math.sqrt(cfg.head_dim)
        nq, nk = q.shape[0], k.shape[0]
        mask = torch.arange(nk, device=self.dev)[None, :] > (q_start + torch.arange(nq, device=self.dev))[:, None]
        s = s.masked_fill(mask[None], float("-inf"))
        return torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), vf).to(torch.bfloat16)

    # ---- the forward pass over `tokens` rows; seqs = [(row_start, row_end, first_position, block_table)] ----------
    def _forward(self, token_ids: torch.Tensor, positions: torch.Tensor, seqs) -> torch.Tensor:
        cfg = self.cfg
        tokens = token_ids.numel()
        delta = self.embed[token_ids.long()].contiguous()                      # what the next norm adds to the residual
        res = torch.zeros(tokens, cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        nq, nkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        for layer in self.layers:
            x_in = delta
            xc, xs = rms_norm_quantize_fp8(delta, layer.g_attn, cfg.eps, residual=res)
            res_attn = res.clone() if self.trace is not None else None
            qkv = layer.qkv.forward(xc, xs)                                    # bf16 [tokens, (nq + 2 nkv) d]
            q = self._rope(qkv[:, : nq * d].reshape(tokens, nq, d), positions)
            k = self._rope(qkv[:, nq * d: (nq + nkv) * d].reshape(tokens, nkv, d), positions)
            v = qkv[:, (nq + nkv) * d:].reshape(tokens, nkv, d)
            attn = torch.empty(tokens, nq, d, dtype=torch.bfloat16, device=self.dev)
            for (r0, r1, p0, table) in seqs:
                new_slots = self._slots(table, p0, p0 + (r1 - r0))
                self._kv_store(layer.k_codes, layer.k_par, k[r0:r1], new_slots)
                self._kv_store(layer.v_codes, layer.v_par, v[r0:r1], new_slots)
                all_slots = self._slots(table, 0, p0 + (r1 - r0))
                attn[r0:r1] = self._attend(q[r0:r1], self._kv_load(layer.k_codes, layer.k_par, all_slots),
                                           self._kv_load(layer.v_codes, layer.v_par, all_slots), p0)
            ac, as_ = self.codec.quantize_rows(attn.view(tokens, nq * d), tokens, nq * d)
            delta = o_out = layer.o.forward(ac.view(tokens, nq * d), as_)
            xc, xs = rms_norm_quantize_fp8(delta, layer.g_mlp, cfg.eps, residual=res)
            gu = layer.gate_up.forward(xc, xs)                                 # gate | up
            hc = torch.empty(tokens, cfg.ffn, dtype=torch.uint8, device=self.dev)
            hs = torch.empty(tokens, dtype=torch.float32, device=self.dev)
            default_handle().call("b2q_swiglu_quantize_rows_bf16", ptr(gu), ptr(gu[:, cfg.ffn:]), tokens, cfg.ffn, 2 * cfg.ffn,
                                  L.FP8_E4M3, L.ROUND_RNE, ptr(hs), ptr(hc))
            delta = layer.down.forward(hc, hs)
            if self.trace is not None:
                self.trace.append(dict(x_in=x_in, res_attn=res_attn, qkv=qkv, attn=attn.clone(), o_out=o_out, res_mlp=res.clone(), gu=gu,
                                       mlp_out=delta))
        xc, xs = rms_norm_quantize_fp8(delta, self.g_final, cfg.eps, residual=res)
        return xc, xs

    def _logits(self, xc: torch.Tensor, xs: torch.Tensor, rows) -> list:
        idx = torch.tensor(rows, device=self.dev, dtype=torch.long)
        out = torch.empty(len(rows), self.cfg.vocab_size, dtype=torch.float32, device=self.dev)
        self.lm_head.forward(xc[idx].contiguous(), xs[idx].contiguous(), out=out)
        return out.cpu().tolist()

    # ---- ModelRunner --------------------------------------------------------------------------------------------
    def decode(self, token_ids, block_tables, seq_lens):
        """model_runner.rs:36-41: one new token per sequence, `seq_lens[i]` tokens already cached."""
        n = len(token_ids)
        _check_batch(n, len(block_tables), len(seq_lens))
        ids = torch.tensor(list(token_ids), device=self.dev, dtype=torch.int32)
        pos = torch.tensor(list(seq_lens), device=self.dev, dtype=torch.long)
        seqs = [(i, i + 1, int(seq_lens[i]), block_tables[i]) for i in range(n)]
        xc, xs = self._forward(ids, pos, seqs)
        return self._logits(xc, xs, list(range(n)))

    def prefill(self, token_ids, seq_starts, block_tables):
        """model_runner.rs:56-61: prompts concatenated in `token_ids`, sequence i is [seq_starts[i], seq_starts[i+1])."""
        if len(token_ids) == 0 or len(seq_starts) < 2:
            raise EmptyBatch(L.ERR_EMPTY_INPUT, "empty batch")
        n = len(seq_starts) - 1
        if n != len(block_tables):
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n}, got {len(block_tables)}")
        if seq_starts[-1] != len(token_ids):
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {seq_starts[-1]}, got {len(token_ids)}")
        ids = torch.tensor(list(token_ids), device=self.dev, dtype=torch.int32)
        pos = torch.cat([torch.arange(seq_starts[i + 1] - seq_starts[i], device=self.dev) for i in range(n)])
        seqs = [(seq_starts[i], seq_starts[i + 1], 0, block_tables[i]) for i in range(n)]
        xc, xs = self._forward(ids, pos, seqs)
        return self._logits(xc, xs, [seq_starts[i + 1] - 1 for i in range(n)])
