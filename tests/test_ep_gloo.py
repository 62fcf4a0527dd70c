"""Expert-parallel dispatch/combine logic on CPU: world_size-2 gloo ranks drive
paramecia_b200.ep.ExpertParallelMoe with the CPU oracle standing in for the GPU block, and the
result must equal the oracle's single-rank block output."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBlock:
    """The MoeBlock surface ExpertParallelMoe uses, served by the CPU oracle on one expert slice."""

    def __init__(self, t, rank, world):
        from tests.common import oracle_layer
        self.full = oracle_layer(t)
        self.num_experts, self.num_experts_per_tok, self.hidden_dim = t["E"], t["k"], t["H"]
        self.num_experts_local = t["E"] // world
        self.expert_base = rank * self.num_experts_local
        self.has_shared = t["shared"] is not None

    def route(self, x, out=None):
        logits = self.full.router_logits(x.float().numpy())
        idx, w = self.full.route_topk(logits)
        res = torch.from_numpy(logits), torch.from_numpy(w), torch.from_numpy(idx.astype(np.int32))
        if out is not None:
            for dst, src in zip(out, res):
                dst.copy_(src)
            return out
        return res

    def experts_forward_batched(self, x, idx, w, top_k, out_dtype=torch.float32, shared_rows=None, out=None):
        ids = idx.numpy().astype(np.int64)
        lo, hi = self.expert_base, self.expert_base + self.num_experts_local
        masked = np.where((ids >= lo) & (ids < hi), ids, 0xFFFFFFFF).astype(np.uint32)  # only this rank's slice
        res = self.full.experts_forward(x.float().numpy(), masked, w.numpy())
        if shared_rows is not None:
            b, c = shared_rows
            res[b:b + c] += self.full.shared_forward(x[b:b + c].float().numpy())
        res = torch.from_numpy(res)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def shared_forward(self, x, out_dtype=torch.float32):
        return torch.from_numpy(self.full.shared_forward(x.float().numpy()))


class NumpyOps:
    @staticmethod
    def reduce_rows(parts, extra, out):
        acc = parts[0].clone()
        for r in range(1, parts.shape[0]):
            acc += parts[r]
        if extra is not None:
            acc += extra
        out.copy_(acc)


def _worker(rank, world, port, mode, ret, k=3):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from paramecia_b200 import synth
        from paramecia_b200.ep import ExpertParallelMoe
        from tests.common import oracle_layer, seeded_x
        t = synth.make_layer(E=8, k=k, preset="q4k_m", seed=2)
        n = 5
        x_all = seeded_x(world * n, 2048, 31)
        x = x_all[rank * n:(rank + 1) * n].contiguous()
        ep = ExpertParallelMoe(OracleBlock(t, rank, world), mode=mode, ops=NumpyOps)
        out = torch.empty((n, 2048), dtype=torch.float32)
        stats = {}
        ep.forward_into(x, out, stats)
        want, _, want_idx, _ = oracle_layer(t).forward(x_all.numpy())
        want = want[rank * n:(rank + 1) * n]
        err = float(np.abs(out.numpy() - want).max() / np.abs(want).max())
        same_idx = bool(np.array_equal(stats["top_indices"].numpy().astype(np.uint32), want_idx[rank * n:(rank + 1) * n]))
        ret[rank] = (err, same_idx)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,k", [("all_to_all", 3), ("all_gather", 3), ("a2av", 3), ("a2av", 1)])
def test_two_ranks_equal_one(mode, k):
    # a2av: the exchange of the native path (exact counts; with k = 1 most tokens stay on one rank)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, mode, ret, k), nprocs=2, join=True)
    assert len(ret) == 2
    for rank in range(2):
        err, same_idx = ret[rank]
        assert same_idx
        assert err < 1e-6, (rank, err)   # fp32 re-association of the cross-rank sum only


def test_four_ranks_equal_one():
    # the all-to-all-v plan with more than one peer: 8 experts over 4 ranks, tokens visit 1 to 3 of them
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(4, port, "a2av", ret, 3), nprocs=4, join=True)
    assert len(ret) == 4
    for rank in range(4):
        err, same_idx = ret[rank]
        assert same_idx and err < 1e-6, (rank, err)


def test_destination_masks():
    from paramecia_b200.ep import INVALID_EXPERT, expert_owner, mask_for_destinations
    idx = torch.tensor([[0, 5, 7], [3, 4, 6]], dtype=torch.int32)
    assert expert_owner(idx, 4).tolist() == [[0, 1, 1], [0, 1, 1]]
    m = mask_for_destinations(idx, 2, 4)
    assert m[0].tolist() == [[0, INVALID_EXPERT, INVALID_EXPERT], [3, INVALID_EXPERT, INVALID_EXPERT]]
    assert m[1].tolist() == [[INVALID_EXPERT, 5, 7], [INVALID_EXPERT, 4, 6]]


def test_dispatch_plan():
    from paramecia_b200.ep import plan_dispatch
    # 4 experts per rank, 2 ranks; rank 0 is home
    idx = torch.tensor([[0, 1], [4, 5], [3, 6], [7, 4], [-1, 2]], dtype=torch.int32)
    pos, cnt = plan_dispatch(idx, 2, 4, self_rank=0)
    assert pos[:, 0].tolist() == [0, 1, 2, 3, 4]            # the home rank takes every token (shared expert)
    assert pos[:, 1].tolist() == [-1, 0, 1, 2, -1]          # rank 1 only the tokens with an expert 4..7
    assert cnt.tolist() == [5, 3]
    pos, cnt = plan_dispatch(idx, 2, 4, self_rank=0, round_robin=True)   # expert e on rank e % 2
    assert pos[:, 1].tolist() == [0, 1, 2, 3, -1] and cnt.tolist() == [5, 4]
    pos, cnt = plan_dispatch(idx, 2, 4, self_rank=1, self_takes_all=False)
    assert pos[:, 0].tolist() == [0, -1, 1, -1, 2] and cnt.tolist() == [3, 3]
