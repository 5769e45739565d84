"""CPU, world_size 2 over gloo: the host-side logic of the tensor-parallel path — rank coordinates, shard
ranges, and that an all-reduce / all-gather of per-rank partials reproduces the reference's rank-ordered
sum / concatenation (RowLinear::all_reduce, ColumnLinear::all_gather) on the same inputs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import api
        from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, column_shard_rows, row_shard_cols
        h = DistInferHandle(rank, ParallelismConfig(tp=world))
        rng = np.random.default_rng(77)                  # same stream on every rank
        batch, hidden, ffn = 3, 64, 96
        x = rng.standard_normal((batch, hidden)).astype(np.float32)
        w_up = (rng.standard_normal((ffn, hidden)) * 0.1).astype(np.float32)
        w_down = (rng.standard_normal((hidden, ffn)) * 0.1).astype(np.float32)
        # column-parallel up projection: this rank's rows, oracle arithmetic on the shard
        r0, r1 = column_shard_rows(ffn, world, h.tp_rank())
        local = api.column_linear(x, w_up[r0:r1], None, batch, hidden, r1 - r0, 1)
        parts = [torch.empty(batch, r1 - r0) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(local))
        gathered = torch.cat(parts, dim=1).numpy()
        full = api.column_linear(x, w_up, None, batch, hidden, ffn, world)
        ok_gather = np.array_equal(gathered, full)       # concatenation: bit-exact
        # row-parallel down projection: this rank's columns of W and of the activation, then all-reduce
        c0, c1 = row_shard_cols(ffn, world, h.tp_rank())
        partial = api.row_linear(full[:, c0:c1], w_down[:, c0:c1], None, batch, c1 - c0, hidden, 1)
        t = torch.from_numpy(partial.copy())
        dist.all_reduce(t)
        ref = api.row_linear(full, w_down, None, batch, ffn, hidden, world)   # sums the partials in rank order
        err = float(np.abs(t.numpy() - ref).max())
        q.put((rank, ok_gather, err, (h.tp_rank(), h.sp_rank(), h.ep_rank())))
    finally:
        dist.destroy_process_group()


def test_tp2_gloo_matches_reference_sharding():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_gather, err, coords in results:
        assert ok_gather, f"rank {rank}: all-gather differs from the rank-ordered concatenation"
        assert err <= 1e-5, f"rank {rank}: all-reduce differs from the rank-ordered sum by {err}"
        assert coords == (rank, 0, 0)
