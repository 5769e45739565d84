"""Worker of tests/test_gpu_tp_mlp.py::test_mlp_tp2_two_ranks: one NCCL rank per GPU."""
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
    from oxicuda_b200.dist_infer import DistInferHandle, ParallelismConfig, TpFp8Mlp
    from test_gpu_tp_mlp import make_inputs, oracle_mlp, rel_err
    tokens, hidden, ffn = 64, 512, 2048
    x, wg, wu, wd = make_inputs(tokens, hidden, ffn)
    t = lambda a: torch.from_numpy(a).to(dev)
    mlp = TpFp8Mlp(t(wg), t(wu), t(wd), DistInferHandle(rank, ParallelismConfig(tp=world)))
    y = mlp.forward(t(x).to(torch.bfloat16)).float().cpu().numpy()
    ref = oracle_mlp(api, x, wg, wu, wd, world)
    err = rel_err(y, ref)
    ok = torch.tensor([1 if err <= 1e-2 else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"rel_err {err:.3e}")
        print("TP2 OK" if int(ok.item()) == 1 else "TP2 FAIL")
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 1)


if __name__ == "__main__":
    main()
