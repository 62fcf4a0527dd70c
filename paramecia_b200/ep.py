"""Expert parallelism for the MoE block: E/N routed experts per GPU, one process per GPU.

The reference is a single-device program (its "expert parallelism" is a rayon loop over
experts, paramecia-model/src/tokio_experts.rs:116-130); the split across GPUs is this build's.
Every rank keeps the router and the shared expert (small) and one contiguous slice of the
routed experts.  One block forward on a rank that is home to n tokens:

1. route the local tokens (router replicated);
2. dispatch: every rank that owns one of a token's experts receives the token's row once,
   with the token's top-k ids and weights; ids the destination does not own are replaced by
   an invalid id so the receiver skips them;
3. each rank runs its experts over what it received and pre-reduces, per token, the weighted
   outputs of its own experts; on its own tokens' rows the same kernels add the shared expert
   (``MoeBlock.experts_forward_batched(..., shared_rows=...)``, ``pmoe_experts_forward_ep``);
4. combine: the per-rank partial rows travel back to the token's home rank and are added there
   (``pmoe_reduce_rows``, rank order) or on the way (reduce-scatter).

Buffers have a fixed capacity of n rows per (source, destination) pair -- a token is sent to a
rank at most once -- so neither exchange needs a size handshake or a host synchronisation.
With top-10 routing over at most 8 ranks nearly every token visits nearly every rank, so the
padding costs little.  Two transports carry the same rows:

* ``all_to_all``  ``all_to_all_single`` calls out (rows, ids, weights) and one back, the sum done by
                  ``pmoe_reduce_rows`` on the home rank;
* ``all_gather``  ``all_gather_into_tensor`` out (the three tensors handed to NCCL as one group, so
                  one launch) and ``reduce_scatter_tensor`` back, which lets NCCL do the cross-rank
                  sum (in the switch when NVLS is active).  With a fixed capacity of n rows per pair
                  both transports move the same bytes; this one needs no send-side packing.

No kernel here reads another GPU's memory: NCCL delivers into local HBM first.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.distributed as dist

INVALID_EXPERT = -1  # 0xFFFFFFFF as int32: outside every expert slice


class _LibOps:
    """The device-side pieces of the combine, from libpmoe."""

    @staticmethod
    def reduce_rows(parts: torch.Tensor, extra: Optional[torch.Tensor], out: torch.Tensor):
        from ._lib import check, lib
        from .moe import _TORCH_TO_PMOE, _stream_ptr
        R, n, H = parts.shape
        check(lib().pmoe_reduce_rows(parts.device.index or 0, parts.data_ptr(), R,
                                     None if extra is None else extra.data_ptr(),
                                     0 if extra is None else _TORCH_TO_PMOE[extra.dtype], n, H, out.data_ptr(),
                                     _TORCH_TO_PMOE[out.dtype], _stream_ptr(parts.device)))


def expert_owner(idx: torch.Tensor, experts_per_rank: int, n_ranks: int = 0, round_robin: bool = False) -> torch.Tensor:
    """Rank that owns each expert id: e // (E/N) under the contiguous placement, e % N under round-robin."""
    if round_robin:
        return torch.remainder(idx, n_ranks)
    return torch.div(idx, experts_per_rank, rounding_mode="floor")


def mask_for_destinations(idx: torch.Tensor, n_ranks: int, experts_per_rank: int, round_robin: bool = False) -> torch.Tensor:
    """[N, n, k] routing tables, one per destination rank: ids the destination does not own become
    INVALID_EXPERT, so that a row contributes on a rank only through that rank's experts."""
    owner = expert_owner(idx, experts_per_rank, n_ranks, round_robin)  # [n, k]
    dest = torch.arange(n_ranks, device=idx.device).view(-1, 1, 1)   # [N, 1, 1]
    return torch.where(owner.unsqueeze(0) == dest, idx.unsqueeze(0), torch.full_like(idx, INVALID_EXPERT).unsqueeze(0))


class ExpertParallelMoe:
    """One MoE block spread over the ranks of `group`.  `block` is this rank's MoeBlock, built with
    its expert slice (expert_base = rank * E/N, E_local = E/N) and max_tokens >= N * n."""

    def __init__(self, block, group=None, mode: str = "all_gather", ops=None):
        if mode not in ("all_to_all", "all_gather"):
            raise ValueError("mode must be 'all_to_all' or 'all_gather'")
        self.block = block
        self.group = group
        self.mode = mode
        self.ops = ops or _LibOps
        self.rank = dist.get_rank(group)
        self.N = dist.get_world_size(group)
        self.E = block.num_experts
        self.k = block.num_experts_per_tok
        self.H = block.hidden_dim
        if self.E % self.N:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        self.per_rank = self.E // self.N
        self.round_robin = getattr(block, "ep_placement", 0) == 1
        if block.num_experts_local != self.per_rank or (not self.round_robin and block.expert_base != self.rank * self.per_rank):
            raise ValueError("block must hold experts [rank*E/N, (rank+1)*E/N), or rank, rank+N, ... (round-robin)")
        self._buf_n = -1
        # NCCL takes several collectives as one group; gloo (CPU tests) runs them one by one
        self._coalesce = dist.get_backend(group) == "nccl"

    # buffers are sized once per token count and reused (no allocation in the steady state)
    def _buffers(self, n: int, x: torch.Tensor):
        if n == self._buf_n and self._x_dtype == x.dtype:
            return
        N, H, k, dev = self.N, self.H, self.k, x.device
        self._buf_n, self._x_dtype = n, x.dtype
        self.logits = torch.empty((n, self.E), dtype=torch.float32, device=dev)
        self.idx = torch.empty((n, k), dtype=torch.int32, device=dev)
        self.w = torch.empty((n, k), dtype=torch.float32, device=dev)
        self.recv_x = torch.empty((N * n, H), dtype=x.dtype, device=dev)
        self.recv_idx = torch.empty((N * n, k), dtype=torch.int32, device=dev)
        self.recv_w = torch.empty((N * n, k), dtype=torch.float32, device=dev)
        self.part = torch.empty((N * n, H), dtype=torch.float32, device=dev)
        self.home = torch.empty((n, H), dtype=torch.float32, device=dev)
        if self.mode == "all_to_all":
            self.send_x = torch.empty((N, n, H), dtype=x.dtype, device=dev)
            self.send_idx = torch.empty((N, n, k), dtype=torch.int32, device=dev)
            self.send_w = torch.empty((N, n, k), dtype=torch.float32, device=dev)
            self.back = torch.empty((N, n, H), dtype=torch.float32, device=dev)

    def gather_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """All ranks' token rows, rank-major: [N*n, H]."""
        out = torch.empty((self.N * x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def _batched(self, device):
        """Context that hands the collectives issued inside it to NCCL as one group (one launch)."""
        if self._coalesce and device.type == "cuda":
            from torch.distributed.distributed_c10d import _coalescing_manager
            return _coalescing_manager(group=self.group, device=device, async_ops=False)
        return contextlib.nullcontext()

    @staticmethod
    def default_mode() -> str:
        return "all_gather"

    def _mark(self, profile, name):
        if profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events[name] = ev

    def trace_experts(self, x: torch.Tensor, reps: int) -> dict:
        """Milliseconds per phase of this rank's expert kernels on the rows a dispatch of `x` delivers."""
        out = torch.empty((x.shape[0], self.H), dtype=torch.bfloat16, device=x.device)
        self.forward_into(x, out)
        n = x.shape[0]
        own = (self.rank * n, n) if self.block.has_shared else None
        acc = {}
        self.block.trace(True)
        for i in range(reps + 3):
            self.block.experts_forward_batched(self.recv_x, self.recv_idx, self.recv_w, self.k, shared_rows=own, out=self.part)
            t = self.block.trace_read()
            if i >= 3:
                for k_, v in t.items():
                    acc[k_] = acc.get(k_, 0.0) + v / reps
        self.block.trace(False)
        return acc

    def forward_into(self, x: torch.Tensor, out: torch.Tensor, stats: Optional[dict] = None, profile: bool = False):
        """x [n, H] (this rank's tokens) -> out [n, H]; every rank must call with the same n.  With `profile` the call
        brackets the dispatch and the combine with CUDA events on the launching stream, waits for them and returns
        {"dispatch", "combine", "total"} in milliseconds."""
        n = x.shape[0]
        N, k, g = self.N, self.k, self.group
        x = x.contiguous()
        self._buffers(n, x)
        self._events = {}
        self._mark(profile, "t0")
        self.block.route(x, out=(self.logits, self.w, self.idx))
        self._mark(profile, "d0")
        if stats is not None:
            stats.update(router_logits=self.logits, top_indices=self.idx, top_weights=self.w)
        # -- dispatch: rows, ids and weights of every token to every rank that may own one of its experts
        if self.mode == "all_to_all":
            self.send_x.copy_(x.unsqueeze(0).expand(N, n, self.H))
            self.send_idx.copy_(mask_for_destinations(self.idx, N, self.per_rank, self.round_robin))
            self.send_w.copy_(self.w.unsqueeze(0).expand(N, n, k))
            dist.all_to_all_single(self.recv_x, self.send_x.view(N * n, self.H), group=g)
            dist.all_to_all_single(self.recv_idx, self.send_idx.view(N * n, k), group=g)
            dist.all_to_all_single(self.recv_w, self.send_w.view(N * n, k), group=g)
        else:
            # ids stay as routed: a rank skips the ids outside its expert slice by itself
            with self._batched(x.device):
                dist.all_gather_into_tensor(self.recv_x, x, group=g)
                dist.all_gather_into_tensor(self.recv_idx, self.idx, group=g)
                dist.all_gather_into_tensor(self.recv_w, self.w, group=g)
        # -- this rank's experts over everything it received, pre-reduced per token.  Rows
        # [rank*n, (rank+1)*n) are this rank's own tokens: the shared expert rides along on those,
        # so each token's shared row is computed once, on its home rank, in the same kernels.
        self._mark(profile, "d1")
        own = (self.rank * n, n) if self.block.has_shared else None
        self.block.experts_forward_batched(self.recv_x, self.recv_idx, self.recv_w, k, shared_rows=own, out=self.part)
        self._mark(profile, "c0")
        # -- combine: the partial rows go back to the token's home rank and are added in rank order
        if self.mode == "all_to_all":
            dist.all_to_all_single(self.back.view(N * n, self.H), self.part, group=g)
            self.ops.reduce_rows(self.back, None, out)
        elif out.dtype == torch.float32 and out.is_contiguous():
            dist.reduce_scatter_tensor(out, self.part, group=g)
        else:
            dist.reduce_scatter_tensor(self.home, self.part, group=g)
            out.copy_(self.home)
        if profile:
            self._mark(True, "c1")
            torch.cuda.synchronize()
            e = self._events
            return dict(dispatch=e["d0"].elapsed_time(e["d1"]), combine=e["c0"].elapsed_time(e["c1"]),
                        total=e["t0"].elapsed_time(e["c1"]))
        return out

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.H), dtype=out_dtype or x.dtype, device=x.device)
        return self.forward_into(x, out)
