"""Worker of tests/test_gpu_moe.py::test_moe_expert_parallel_two_ranks: one NCCL rank per GPU, each owning half of
the experts; the layer's result on every rank against the oracle composition of router, dispatcher and SwiGLU experts."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from oracle import api
    api.set_threads(max(1, len(os.sched_getaffinity(0)) // world))
    from oxicuda_b200._lib import default_handle
    from oxicuda_b200.dist_infer import DistInferHandle, MoeFp8Layer, ParallelismConfig
    from test_gpu_moe import _bf16, err, oracle_moe
    tokens, n_experts, top_k, hidden, ffn = 300, 8, 2, 256, 512
    rng = np.random.default_rng(0xB2000004)                     # the same stream on every rank
    x = _bf16(rng.standard_normal((tokens, hidden)))
    logits = rng.standard_normal((tokens, n_experts)).astype(np.float32)
    experts = [((rng.standard_normal((ffn, hidden)) * 0.02).astype(np.float32),
                (rng.standard_normal((ffn, hidden)) * 0.02).astype(np.float32),
                (rng.standard_normal((hidden, ffn)) * 0.02).astype(np.float32)) for _ in range(n_experts)]
    ref, idx, _ = oracle_moe(api, x, logits, experts, top_k)
    t = lambda a: torch.from_numpy(a).to(dev)
    local = n_experts // world
    mine = experts[rank * local:(rank + 1) * local]
    layer = MoeFp8Layer([(t(a), t(b), t(c)) for a, b, c in mine], n_experts, top_k, DistInferHandle(rank, ParallelismConfig(ep=world)))
    y = layer.forward(t(x).to(torch.bfloat16), t(logits)).float().cpu().numpy()
    default_handle().check()
    e = err(y, ref)
    counts_ok = np.array_equal(layer.last_counts.cpu().numpy(), np.bincount(idx.reshape(-1), minlength=n_experts)[rank * local:(rank + 1) * local])
    ok = torch.tensor([1 if e <= 1e-2 and counts_ok else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"rel_err {e:.3e}, counts_ok {counts_ok}")
        print("EP2 OK" if int(ok.item()) == 1 else "EP2 FAIL")
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 1)


if __name__ == "__main__":
    main()
