"""Host-side mirror of oxicuda-dist-infer's tensor-parallel linears, one process per GPU.

The reference simulates ranks in one thread and its collectives are Vec sums
(`crates/oxicuda-dist-infer/src/tensor_parallel/{column,row}_parallel.rs`); here each rank is a
process on its own GPU, shards are quantized weights in HBM, the matmuls are the FP8 kernels of
libb2q and the boundary collectives run inside libb2q (b2q_tp_*, include/b2q.h): a peer-memory all-reduce kernel for few tokens,
NCCL overlapped with the GEMMs for many; torch.distributed only carries the set-up messages.
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


class TpGroup:
    """b2q_tp (include/b2q.h): the library handle bound to an NCCL communicator of the tp ranks, a second stream for
    overlapped collectives and the peer-mapped exchange buffers of the few-token all-reduce kernel.

    The communicator is created here through the library's own helpers: rank 0 of the group draws the NCCL unique
    id, torch.distributed carries it (and the CUDA IPC handles of the exchange buffers) to the other ranks."""

    def __init__(self, handle: DistInferHandle, attach_peers: bool = True):
        import ctypes as C
        self.handle = handle
        self.tp, self.rank = handle.config.tp, handle.tp_rank()
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._lib = L.lib()
        self._h = L.default_handle()
        self._comm = C.c_void_p(0)
        self._t = C.c_void_p(0)
        group = handle.group
        if self.tp > 1:
            src = dist.get_global_rank(group, 0) if group is not None else 0
            ident = torch.zeros(128, dtype=torch.uint8, device=self.device)
            if self.rank == 0:
                buf = (C.c_uint8 * 128)()
                self._check(self._lib.b2q_tp_unique_id(buf), "b2q_tp_unique_id")
                ident.copy_(torch.frombuffer(bytearray(buf), dtype=torch.uint8))
            dist.broadcast(ident, src=src, group=group)
            idb = (C.c_uint8 * 128).from_buffer_copy(bytes(ident.cpu().numpy().tobytes()))
            self._check(self._lib.b2q_tp_comm_init(idb, self.tp, self.rank, C.byref(self._comm)), "b2q_tp_comm_init")
        st = self._lib.b2q_tp_create(self._h._h, self._comm, self.tp, self.rank, C.byref(self._t))
        self._check(st, "b2q_tp_create")
        self.peers_attached = False
        if self.tp > 1 and attach_peers:
            hd = (C.c_uint8 * 64)()
            self._check(self._lib.b2q_tp_exchange_buffer(self._t, None, hd), "b2q_tp_exchange_buffer")
            mine = torch.frombuffer(bytearray(hd), dtype=torch.uint8).to(self.device)
            every = [torch.empty_like(mine) for _ in range(self.tp)]
            dist.all_gather(every, mine, group=group)
            flat = b"".join(bytes(t.cpu().numpy().tobytes()) for t in every)
            arr = (C.c_uint8 * len(flat)).from_buffer_copy(flat)
            self._check(self._lib.b2q_tp_attach_peers(self._t, arr, None), "b2q_tp_attach_peers")
            self.peers_attached = True

    def _check(self, st: int, what: str):
        if st != L.OK:
            msg = self._lib.b2q_last_error(self._h._h)
            raise L._ERRORS.get(st, L.B2qError)(st, (msg.decode() if msg else "") or what)

    def call(self, name: str, *args):
        L.default_handle()                                   # the handle follows torch's current stream
        self._check(getattr(self._lib, name)(self._t, *args), name)

    def set_chunks(self, chunks: int):
        self.call("b2q_tp_set_chunks", chunks)

    def plan(self, tokens: int, out_features: int):
        """(mode, chunks) of b2q_tp_plan for a row-parallel result of this shape."""
        import ctypes as C
        mode, chunks = C.c_int(0), C.c_int(0)
        st = self._lib.b2q_tp_plan(self.tp, 1 if self.peers_attached else 0, tokens, out_features, C.byref(mode), C.byref(chunks))
        self._check(st, "b2q_tp_plan")
        return mode.value, chunks.value

    def close(self):
        if getattr(self, "_t", None) and self._t.value:
            torch.cuda.synchronize()
            self._lib.b2q_tp_destroy(self._t)
            self._t.value = 0
        if getattr(self, "_comm", None) and self._comm.value:
            self._lib.b2q_tp_comm_destroy(self._comm)
            self._comm.value = 0


_groups = {}


def tp_group(handle: DistInferHandle) -> TpGroup:
    """One TpGroup per (process group, tp, rank, device), created on first use (a collective call when tp > 1)."""
    key = (id(handle.group), handle.config.tp, handle.tp_rank(), torch.cuda.current_device())
    g = _groups.get(key)
    if g is None:
        g = _groups[key] = TpGroup(handle)
    return g


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
    """ColumnLinear (column_parallel.rs:103-205): this rank owns out/tp consecutive rows of W[out x in] and of the bias."""

    def __init__(self, full_weight: torch.Tensor, handle: DistInferHandle, rounding: str = "rne", bias: torch.Tensor = None):
        self.handle = handle
        self.total_out = full_weight.shape[0]
        r0, r1 = column_shard_rows(self.total_out, handle.config.tp, handle.tp_rank())
        self.shard = Fp8Linear(full_weight[r0:r1], rounding)
        self.bias = None if bias is None else bias[r0:r1].float().contiguous()

    def forward(self, x_codes, x_scales, gather: bool = False) -> torch.Tensor:
        """b2q_column_linear_forward: the local output [tokens x out/tp], or with gather=True the gathered
        [tokens x out] (column_parallel.rs:181-204: shard r lands at columns [r*out/tp, ...))."""
        tokens = x_codes.shape[0]
        local = torch.empty(tokens, self.shard.out_features, dtype=torch.bfloat16, device=x_codes.device)
        full = torch.empty(tokens, self.total_out, dtype=torch.bfloat16, device=x_codes.device) if gather else None
        tp_group(self.handle).call("b2q_column_linear_forward", L.ptr(x_codes), L.ptr(x_scales), L.ptr(self.shard.codes),
                                   L.ptr(self.shard.scales), L.ptr(self.bias), tokens, self.shard.in_features,
                                   self.shard.out_features, L.ptr(local), L.ptr(full))
        return full if gather else local

    def local_forward(self, x_codes, x_scales) -> torch.Tensor:
        return self.forward(x_codes, x_scales)

    def all_gather(self, local: torch.Tensor) -> torch.Tensor:
        """column_parallel.rs:181-204 on an existing local result (torch.distributed)."""
        tp = self.handle.config.tp
        if tp == 1:
            return local
        parts = [torch.empty_like(local) for _ in range(tp)]
        dist.all_gather(parts, local, group=self.handle.group)
        return torch.cat(parts, dim=1)


class RowLinear:
    """RowLinear (row_parallel.rs:97-224): this rank owns in/tp consecutive columns of every row; the bias is added
    on rank 0 only (row_parallel.rs:183-190)."""

    def __init__(self, full_weight: torch.Tensor, handle: DistInferHandle, rounding: str = "rne", bias: torch.Tensor = None):
        self.handle = handle
        self.total_in = full_weight.shape[1]
        c0, c1 = row_shard_cols(self.total_in, handle.config.tp, handle.tp_rank())
        self.cols = (c0, c1)
        self.shard = Fp8Linear(full_weight[:, c0:c1].contiguous(), rounding)
        self.bias = None if bias is None else bias.float().contiguous()

    def forward(self, x_codes, x_scales, out: torch.Tensor = None) -> torch.Tensor:
        """b2q_row_linear_forward_allreduce: x_codes is this rank's column slice [tokens x in/tp]; returns the sum over
        ranks [tokens x out] (peer-memory kernel for few tokens, chunked NCCL all-reduce overlapped with the GEMM
        otherwise; neither sums in NCCL's order nor bit for bit in the host's, hence a tolerance in the tests)."""
        tokens = x_codes.shape[0]
        y = out if out is not None else torch.empty(tokens, self.shard.out_features, dtype=torch.bfloat16, device=x_codes.device)
        tp_group(self.handle).call("b2q_row_linear_forward_allreduce", L.ptr(x_codes), L.ptr(x_scales), L.ptr(self.shard.codes),
                                   L.ptr(self.shard.scales), L.ptr(self.bias), tokens, self.shard.in_features,
                                   self.shard.out_features, L.ptr(y))
        return y

    def forward_partial(self, x_codes, x_scales, out=None) -> torch.Tensor:
        return self.shard.forward(x_codes, x_scales, out=out)

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """row_parallel.rs:202-223 on an existing partial, in place (NCCL on the handle's stream)."""
        if self.handle.config.tp > 1:
            tp_group(self.handle).call("b2q_tp_all_reduce_bf16", L.ptr(partial), partial.numel())
        return partial


class TpFp8Mlp:
    """Tensor-parallel SwiGLU MLP with FP8 weights: gate and up column-parallel (fused into one GEMM over the
    concatenated shard), down row-parallel, the sum over ranks after the down projection
    (b2q_mlp_swiglu_fp8_forward).

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
        self._interleave()

    @classmethod
    def from_shards(cls, w_gate_shard: torch.Tensor, w_up_shard: torch.Tensor, w_down_shard: torch.Tensor,
                    handle: DistInferHandle, rounding: str = "rne"):
        """Builds the layer from this rank's slices only: gate/up rows [ffn/tp x hidden], down columns [hidden x ffn/tp]."""
        self = cls.__new__(cls)
        self.handle = handle
        self.local_ffn, self.hidden = w_gate_shard.shape
        self.gate_up = Fp8Linear(torch.cat([w_gate_shard, w_up_shard], dim=0), rounding)
        self.down = Fp8Linear(w_down_shard.contiguous(), rounding)
        self.codec = Fp8Codec.e4m3(rounding)
        self._interleave()
        return self

    def _interleave(self):
        """Load-time step: the gate and up rows (codes and scales) interleaved per 128 rows (b2q_interleave_rows128), the
        layout whose GEMM tiles hold both projections of the same hidden units so that forward() forms silu(gate) * up in
        the GEMM epilogue.  Shards whose width is not a multiple of 128 keep the concatenated layout."""
        from ._lib import default_handle, ptr
        F = self.local_ffn
        self.gu_codes = self.gu_scales = None
        if F % 128 != 0 or self.hidden % 16 != 0:
            return
        codes, scales = self.gate_up.codes, self.gate_up.scales
        self.gu_codes, self.gu_scales = torch.empty_like(codes), torch.empty_like(scales)
        h = default_handle()
        h.call("b2q_interleave_rows128", ptr(codes), ptr(codes[F:]), F, self.hidden, ptr(self.gu_codes))
        h.call("b2q_interleave_rows128", ptr(scales), ptr(scales[F:]), F, 4, ptr(self.gu_scales))

    def forward_partial(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [tokens x hidden] (replicated) -> this rank's partial of the output, bf16 [tokens x hidden]
        (separate library calls; forward() is the fused entry point)."""
        from ._lib import default_handle, ptr
        tokens = x.shape[0]
        xc, xs = self.codec.quantize_rows(x, tokens, self.hidden)
        F = self.local_ffn
        if self.gu_codes is not None:                                            # interleaved layout: h leaves the GEMM epilogue as bf16
            from .blas import EpilogueOp, gemm_fp8_ex
            h = gemm_fp8_ex(xc.view(tokens, self.hidden), self.gu_codes, xs, self.gu_scales, epilogue=EpilogueOp.SwiGluPairs)
            hc, hs = self.codec.quantize_rows(h, tokens, F)
            return self.down.forward(hc.view(tokens, F), hs)
        gu = self.gate_up.forward(xc.view(tokens, self.hidden), xs)              # bf16 [tokens x 2F]: gate | up
        hc = torch.empty(tokens, F, dtype=torch.uint8, device=x.device)
        hs = torch.empty(tokens, dtype=torch.float32, device=x.device)
        default_handle().call("b2q_swiglu_quantize_rows_bf16", ptr(gu), ptr(gu[:, F:]), tokens, F, 2 * F,
                              L.FP8_E4M3, self.codec.rounding, ptr(hs), ptr(hc))
        return self.down.forward(hc, hs)

    def forward(self, x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        tokens = x.shape[0]
        y = out if out is not None else torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=x.device)
        inter = self.gu_codes is not None
        tp_group(self.handle).call("b2q_mlp_swiglu_fp8_forward_ex", L.ptr(x), L.ptr(self.gu_codes if inter else self.gate_up.codes),
                                   L.ptr(self.gu_scales if inter else self.gate_up.scales), L.ptr(self.down.codes), L.ptr(self.down.scales),
                                   tokens, self.hidden, self.local_ffn, self.codec.rounding,
                                   L.GATE_UP_INTERLEAVED128 if inter else L.GATE_UP_CONCATENATED, L.ptr(y))
        return y


@dataclass
class RoutingPlan:
    """RoutingPlan, crates/oxicuda-dist-infer/src/expert_parallel/router.rs:12-60: per token the top-k experts
    (descending logit) and the softmax of those k logits."""
    expert_idx: torch.Tensor      # int32 [tokens x top_k]
    weight: torch.Tensor          # f32   [tokens x top_k]
    expert_load: torch.Tensor     # int64 [n_experts]
    n_tokens: int
    n_experts: int
    top_k: int


class TopKRouter:
    """TopKRouter::route, crates/oxicuda-dist-infer/src/expert_parallel/router.rs:94-140 (stable descending sort,
    softmax over the selected logits) as one kernel (b2q_moe_route_topk)."""

    def __init__(self, n_experts: int, top_k: int):
        if top_k < 1 or top_k > n_experts:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"top_k {top_k} must be in [1, {n_experts}]")
        self.n_experts, self.top_k = n_experts, top_k

    def route(self, logits: torch.Tensor, n_tokens: int) -> RoutingPlan:
        if logits.numel() != n_tokens * self.n_experts:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n_tokens * self.n_experts}, got {logits.numel()}")
        lg = logits.reshape(n_tokens, self.n_experts).float().contiguous()
        idx = torch.empty(n_tokens, self.top_k, dtype=torch.int32, device=lg.device)
        w = torch.empty(n_tokens, self.top_k, dtype=torch.float32, device=lg.device)
        L.default_handle().call("b2q_moe_route_topk", L.ptr(lg), n_tokens, self.n_experts, self.top_k, L.ptr(idx), L.ptr(w))
        load = torch.bincount(idx.reshape(-1).long(), minlength=self.n_experts)
        return RoutingPlan(idx, w, load, n_tokens, self.n_experts, self.top_k)


class MoeFp8Layer:
    """Mixture of SwiGLU experts with FP8 weights, experts sharded across ranks (expert parallel), as one library call
    (b2q_moe_forward): no host synchronisation between routing and the result.

    ExpertDispatcher::dispatch_and_gather (crates/oxicuda-dist-infer/src/expert_parallel/dispatch.rs:99-219) with
    SwiGluExpert::forward (crates/oxicuda-moe/src/expert/ffn.rs:172-243) as the expert: this rank owns experts
    [ep_rank*E/ep, (ep_rank+1)*E/ep); tokens are replicated, every rank computes the pairs routed to its experts
    (route -> slot -> scatter -> per-token FP8 quantize -> ONE grouped gate|up GEMM -> SwiGLU + re-quantize -> ONE grouped
    down GEMM -> weighted gather) and one all-reduce adds the ranks' contributions."""

    def __init__(self, experts, n_experts: int, top_k: int, handle: DistInferHandle, rounding: str = "rne"):
        """experts: list of (w1 gate [ffn x hidden], w3 up [ffn x hidden], w2 down [hidden x ffn]) for THIS rank's experts."""
        ep = handle.config.ep
        if n_experts % ep != 0:
            raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"n_experts {n_experts} not divisible by ep {ep}")
        self.handle, self.n_experts, self.top_k = handle, n_experts, top_k
        self.local = n_experts // ep
        self.first = handle.ep_rank() * self.local
        if len(experts) != self.local:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {self.local} local experts, got {len(experts)}")
        self.ffn, self.hidden = experts[0][0].shape
        gate_up = [Fp8Linear(torch.cat([w1, w3], dim=0), rounding) for (w1, w3, _) in experts]
        down = [Fp8Linear(w2.contiguous(), rounding) for (_, _, w2) in experts]
        # the experts' codes and scales stacked: [E/ep][2*ffn][hidden] and [E/ep][hidden][ffn], the grouped GEMM's operand
        # gate and up rows interleaved per 128 where the width allows it (the SwiGLU epilogue of the grouped GEMM)
        self.interleaved = self.ffn % 128 == 0 and self.hidden % 16 == 0
        if self.interleaved:
            from ._lib import default_handle, ptr
            F, hd = self.ffn, default_handle()
            for g in gate_up:
                codes, scales = torch.empty_like(g.codes), torch.empty_like(g.scales)
                hd.call("b2q_interleave_rows128", ptr(g.codes), ptr(g.codes[F:]), F, self.hidden, ptr(codes))
                hd.call("b2q_interleave_rows128", ptr(g.scales), ptr(g.scales[F:]), F, 4, ptr(scales))
                g.codes, g.scales = codes, scales
        self.gate_up_codes = torch.stack([g.codes for g in gate_up]).contiguous()
        self.gate_up_scales = torch.cat([g.scales for g in gate_up]).contiguous()
        self.down_codes = torch.stack([d.codes for d in down]).contiguous()
        self.down_scales = torch.cat([d.scales for d in down]).contiguous()
        self.router = TopKRouter(n_experts, top_k)
        self.codec = Fp8Codec.e4m3(rounding)
        # the expert-parallel group: the library's rank group over the ep ranks
        self._group_handle = DistInferHandle(handle.ep_rank(), ParallelismConfig(tp=ep), handle.group)
        self.last_counts = None

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """x bf16 [tokens x hidden], logits f32 [tokens x n_experts] -> bf16 [tokens x hidden]."""
        tokens = x.shape[0]
        y = out if out is not None else torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=x.device)
        lg = logits.reshape(tokens, self.n_experts).float().contiguous()
        if self.last_counts is None:
            self.last_counts = torch.zeros(self.local, dtype=torch.int32, device=x.device)
        tp_group(self._group_handle).call("b2q_moe_forward_ex", L.ptr(x), L.ptr(lg), L.ptr(self.gate_up_codes), L.ptr(self.gate_up_scales),
                                          L.ptr(self.down_codes), L.ptr(self.down_scales), tokens, self.hidden, self.ffn, self.n_experts,
                                          self.top_k, self.codec.rounding,
                                          L.GATE_UP_INTERLEAVED128 if self.interleaved else L.GATE_UP_CONCATENATED, L.ptr(y), L.ptr(self.last_counts))
        return y


class MoeFp4Layer:
    """The mixture of SwiGLU experts with block-scaled FP4 weights (E2M1 codes, E8M0 scale per 32 along K), one library
    call (b2q_moe_forward_fp4): routing, slotting and scatter on the device, ONE grouped tcgen05 block-scaled GEMM for
    gate | up, silu(gate) * up in bf16, ONE grouped GEMM for down, weighted gather; expert parallel like MoeFp8Layer.

    Reference items: ExpertDispatcher::dispatch_and_gather (crates/oxicuda-dist-infer/src/expert_parallel/dispatch.rs:99-219),
    SwiGluExpert::forward (crates/oxicuda-moe/src/expert/ffn.rs:172-243), MicroScalingQuantizer
    (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:746-898)."""

    def __init__(self, experts, n_experts: int, top_k: int, handle: DistInferHandle, mxfp8_activations: bool = True):
        """experts: list of (w1 gate [ffn x hidden], w3 up [ffn x hidden], w2 down [hidden x ffn]) f32 for THIS rank's experts."""
        from .blas import MicroScalingConfig, MicroScalingQuantizer, ScalingFormat
        ep = handle.config.ep
        if n_experts % ep != 0:
            raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"n_experts {n_experts} not divisible by ep {ep}")
        self.handle, self.n_experts, self.top_k = handle, n_experts, top_k
        self.local = n_experts // ep
        if len(experts) != self.local:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {self.local} local experts, got {len(experts)}")
        self.ffn, self.hidden = experts[0][0].shape
        msq = MicroScalingQuantizer(MicroScalingConfig(32, ScalingFormat.E8M0))
        gu = [msq.quantize_fp4(torch.cat([w1, w3], dim=0).reshape(-1).float().contiguous()) for (w1, w3, _) in experts]
        dn = [msq.quantize_fp4(w2.reshape(-1).float().contiguous()) for (_, _, w2) in experts]
        self.gate_up_codes = torch.cat([c.reshape(-1) for c, _ in gu]).contiguous()
        self.gate_up_scales = torch.cat([s.reshape(-1) for _, s in gu]).contiguous()
        self.down_codes = torch.cat([c.reshape(-1) for c, _ in dn]).contiguous()
        self.down_scales = torch.cat([s.reshape(-1) for _, s in dn]).contiguous()
        self.act_mode = 1 if mxfp8_activations else 0
        self._group_handle = DistInferHandle(handle.ep_rank(), ParallelismConfig(tp=ep), handle.group)
        self.last_counts = None

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        tokens = x.shape[0]
        y = out if out is not None else torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=x.device)
        lg = logits.reshape(tokens, self.n_experts).float().contiguous()
        if self.last_counts is None:
            self.last_counts = torch.zeros(self.local, dtype=torch.int32, device=x.device)
        tp_group(self._group_handle).call("b2q_moe_forward_fp4", L.ptr(x), L.ptr(lg), L.ptr(self.gate_up_codes), L.ptr(self.gate_up_scales),
                                          L.ptr(self.down_codes), L.ptr(self.down_scales), tokens, self.hidden, self.ffn, self.n_experts,
                                          self.top_k, self.act_mode, L.ptr(y), L.ptr(self.last_counts))
        return y
