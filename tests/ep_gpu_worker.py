"""Worker of tests/test_gpu_ep.py: one rank per GPU, NCCL.  Every rank builds the same seeded
layer, keeps its expert slice, runs the expert-parallel forward on its share of the tokens and
compares with the whole block evaluated on one GPU (rank-local copy of the full layer)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "native"
    placement = sys.argv[2] if len(sys.argv) > 2 else "contiguous"
    preset = sys.argv[3] if len(sys.argv) > 3 else "q4k_m"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from paramecia_b200 import synth
    from paramecia_b200.ep import ExpertParallelMoe
    from tests.common import seeded_x
    E, k, n = 64, 6, 24
    t = synth.make_layer(E=E, k=k, preset=preset, seed=4)
    whole = synth.make_block(t, dev, max_tokens=world * n)
    mine = synth.make_rank_block(t, dev, world * n, rank, world, placement)
    x_all = seeded_x(world * n, 2048, 77, torch.bfloat16).to(dev)
    x = x_all[rank * n:(rank + 1) * n].contiguous()
    ep = ExpertParallelMoe(mine, mode=mode)
    out = torch.empty((n, 2048), dtype=torch.float32, device=dev)
    stats = {}
    ep.forward_into(x, out, stats)
    ep.forward_into(x, out, stats)  # twice: buffers are reused
    want, (_, want_idx) = whole.forward_with_stats(x_all, out_dtype=torch.float32)
    want = want[rank * n:(rank + 1) * n]
    torch.cuda.synchronize()
    mine.status(); whole.status()
    err = float((out - want).abs().max() / want.abs().max())
    ok_idx = bool(torch.equal(stats["top_indices"], want_idx[rank * n:(rank + 1) * n]))
    flag = torch.tensor([1.0 if (err < 1e-5 and ok_idx) else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"EP_RESULT mode={mode} placement={placement} preset={preset} world={world} max_rel_err={err:.3e} "
              f"idx_equal={ok_idx} all_ok={int(flag.item())}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
