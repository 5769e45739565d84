"""Host-side mirror of oxicuda-dist-infer's tensor-parallel linears, one process per GPU.

The reference simulates ranks in one thread and its collectives are Vec sums
(`crates/oxicuda-dist-infer/src/tensor_parallel/{column,row}_parallel.rs`); here each rank is a
process on its own GPU, shards are quantized weights in HBM, the matmuls are the FP8 kernels of
libb2q and the only collective is one NCCL all-reduce (row-parallel boundary) or all-gather
(column-parallel boundary) over NVLink, issued through torch.distributed.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib as L
from .blas import gemm_fp8
from .quant import Fp8Codec


@dataclass
class ParallelismConfig:
    """crates/oxicuda-dist-infer/src/handle.rs:17-60"""
    tp: int = 1
    sp: int = 1
    ep: int = 1

    def world_size(self) -> int:
        return self.tp * self.sp * self.ep


class DistInferHandle:
    """DistInferHandle, crates/oxicuda-dist-infer/src/handle.rs:62-239: rank -> (tp, sp, ep) coordinates."""

    def __init__(self, global_rank: int, config: ParallelismConfig, group=None):
        if config.tp < 1 or config.sp < 1 or config.ep < 1:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, "parallelism degrees must be >= 1")
        if not 0 <= global_rank < config.world_size():
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"rank {global_rank} outside world {config.world_size()}")
        self.global_rank, self.config, self.group = global_rank, config, group

    def tp_rank(self) -> int:
        return self.global_rank % self.config.tp

    def sp_rank(self) -> int:
        return (self.global_rank // self.config.tp) % self.config.sp

    def ep_rank(self) -> int:
        return self.global_rank // (self.config.tp * self.config.sp)


def column_shard_rows(out_features: int, tp: int, rank: int):
    """ColumnLinear::from_full_weight row range, column_parallel.rs:115-166."""
    if out_features % tp != 0:
        raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"out_features {out_features} not divisible by tp {tp}")
    lo = out_features // tp
    return rank * lo, (rank + 1) * lo


def row_shard_cols(in_features: int, tp: int, rank: int):
    """RowLinear::from_full_weight column range, row_parallel.rs:109-168."""
    if in_features % tp != 0:
        raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"in_features {in_features} not divisible by tp {tp}")
    li = in_features // tp
    return rank * li, (rank + 1) * li


class Fp8Linear:
    """One shard of a linear layer held as E4M3 codes with per-output-row scales.
    forward(x_codes, x_scales) -> bf16 [tokens x local_out]."""

    def __init__(self, weight: torch.Tensor, rounding: str = "rne"):
        out_f, in_f = weight.shape
        codec = Fp8Codec.e4m3(rounding)
        codes, scales = codec.quantize_rows(weight.contiguous(), out_f, in_f)
        self.codes = codes.view(out_f, in_f)
        self.scales = scales
        self.out_features, self.in_features = out_f, in_f

    def forward(self, x_codes: torch.Tensor, x_scales: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        return gemm_fp8(x_codes, self.codes, x_scales, self.scales, out=out)


class ColumnLinear:
    """ColumnLinear (column_parallel.rs:103-205): this rank owns out/tp consecutive rows of W[out x in]."""

    def __init__(self, full_weight: torch.Tensor, handle: DistInferHandle, rounding: str = "rne"):
        self.handle = handle
        self.total_out = full_weight.shape[0]
        r0, r1 = column_shard_rows(self.total_out, handle.config.tp, handle.tp_rank())
        self.shard = Fp8Linear(full_weight[r0:r1], rounding)

    def local_forward(self, x_codes, x_scales) -> torch.Tensor:
        return self.shard.forward(x_codes, x_scales)

    def all_gather(self, local: torch.Tensor) -> torch.Tensor:
        """column_parallel.rs:181-204: shard r lands at columns [r*out/tp, ...)."""
        tp = self.handle.config.tp
        if tp == 1:
            return local
        parts = [torch.empty_like(local) for _ in range(tp)]
        dist.all_gather(parts, local, group=self.handle.group)
        return torch.cat(parts, dim=1)


class RowLinear:
    """RowLinear (row_parallel.rs:97-224): this rank owns in/tp consecutive columns of every row."""

    def __init__(self, full_weight: torch.Tensor, handle: DistInferHandle, rounding: str = "rne"):
        self.handle = handle
        self.total_in = full_weight.shape[1]
        c0, c1 = row_shard_cols(self.total_in, handle.config.tp, handle.tp_rank())
        self.cols = (c0, c1)
        self.shard = Fp8Linear(full_weight[:, c0:c1].contiguous(), rounding)

    def forward_partial(self, x_codes, x_scales, out=None) -> torch.Tensor:
        return self.shard.forward(x_codes, x_scales, out=out)

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """row_parallel.rs:202-223 sums partials in rank order; NCCL's order differs, so results agree
        to a tolerance, not bit for bit."""
        if self.handle.config.tp > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.handle.group)
        return partial


class TpFp8Mlp:
    """Tensor-parallel SwiGLU MLP with FP8 weights: gate and up column-parallel (fused into one GEMM over the
    concatenated shard), down row-parallel, one all-reduce after the down projection.

    Semantics: SwiGluExpert::forward (crates/oxicuda-moe/src/expert/ffn.rs:208-243) with the linears sharded as
    ColumnLinear / RowLinear do (crates/oxicuda-dist-infer/src/tensor_parallel/*.rs).  Activations are quantized
    per token (absmax/448), weights per output row; the SwiGLU result is re-quantized per token over this rank's
    columns before the down projection."""

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, handle: DistInferHandle,
                 rounding: str = "rne"):
        self.handle = handle
        tp, r = handle.config.tp, handle.tp_rank()
        ffn, hidden = w_gate.shape
        r0, r1 = column_shard_rows(ffn, tp, r)
        c0, c1 = row_shard_cols(ffn, tp, r)
        self.local_ffn, self.hidden = r1 - r0, hidden
        self.gate_up = Fp8Linear(torch.cat([w_gate[r0:r1], w_up[r0:r1]], dim=0), rounding)   # [2*ffn/tp x hidden]
        self.down = Fp8Linear(w_down[:, c0:c1].contiguous(), rounding)                          # [hidden x ffn/tp]
        self.codec = Fp8Codec.e4m3(rounding)

    def forward_partial(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [tokens x hidden] (replicated) -> this rank's partial of the output, bf16 [tokens x hidden]."""
        from ._lib import default_handle, ptr
        tokens = x.shape[0]
        xc, xs = self.codec.quantize_rows(x, tokens, self.hidden)
        gu = self.gate_up.forward(xc.view(tokens, self.hidden), xs)              # bf16 [tokens x 2F]: gate | up
        F = self.local_ffn
        hc = torch.empty(tokens, F, dtype=torch.uint8, device=x.device)
        hs = torch.empty(tokens, dtype=torch.float32, device=x.device)
        default_handle().call("b2q_swiglu_quantize_rows_bf16", ptr(gu), ptr(gu[:, F:]), tokens, F, 2 * F,
                              L.FP8_E4M3, self.codec.rounding, ptr(hs), ptr(hc))
        return self.down.forward(hc, hs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.forward_partial(x)
        if self.handle.config.tp > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.handle.group)
        return y
