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

* ``native``      (default on GPUs) the whole forward behind the C ABI, ``pmoe_ep_forward``: the dispatch is an
                  all-to-all-v of QUANTISED rows over grouped ncclSend / ncclRecv -- a row travels only to the ranks
                  that hold one of its experts (exact counts, from 2048 rows in flight) or to every rank with the
                  foreign ids masked (padded counts, no host synchronisation) -- and each rank returns one
                  pre-reduced f32 row per record; ``native_exact`` / ``native_padded`` force one of the two.  The
                  library opens its own NCCL communicator from an id this module broadcasts over ``torch.distributed``.

``plan_dispatch`` / ``A2avReference`` restate the native path's index arithmetic (which token goes where, at which
position, and how the returned rows are added) in torch, so that it can be checked on CPU ranks.

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


_NATIVE_MODES = {"native": 0, "native_padded": 1, "native_exact": 2}
_native_comms = {}


def native_comm(group, device: torch.device):
    """The library's own NCCL communicator over the ranks of `group` (one per group and device, created on first use:
    rank 0 makes the id, torch.distributed carries it to the others, every rank joins)."""
    import ctypes as C
    from ._lib import check, lib
    key = (id(group), device.index)
    if key in _native_comms:
        return _native_comms[key]
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    buf = (C.c_ubyte * 128)()
    if rank == 0:
        check(lib().pmoe_ep_unique_id(buf, 128))
    t = torch.tensor(list(buf), dtype=torch.uint8, device=device if dist.get_backend(group) == "nccl" else "cpu")
    dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    raw = bytes(t.cpu().tolist())
    comm = C.c_void_p()
    with torch.cuda.device(device):
        check(lib().pmoe_ep_comm_create(raw, 128, rank, size, device.index, C.byref(comm)))
    _native_comms[key] = comm
    return comm


def plan_dispatch(idx: torch.Tensor, n_ranks: int, experts_per_rank: int, self_rank: int, round_robin: bool = False,
                  self_takes_all: bool = True):
    """The dispatch plan of the native path for one rank's routing table idx [n, k]: ``pos`` [n, N] = position of token
    t among the records for rank r (token order), -1 when t does not travel there; ``cnt`` [N] records per rank.  The
    home rank takes all its tokens (the shared expert runs there)."""
    owner = expert_owner(idx.long(), experts_per_rank, n_ranks, round_robin)             # [n, k]
    valid = (idx.long() >= 0) & (idx.long() < n_ranks * experts_per_rank)
    dest = torch.arange(n_ranks, device=idx.device).view(1, -1, 1)                         # [1, N, 1]
    flag = ((owner.unsqueeze(1) == dest) & valid.unsqueeze(1)).any(-1)                     # [n, N]
    if self_takes_all:
        flag[:, self_rank] = True
    pos = torch.cumsum(flag.long(), 0) - 1
    pos = torch.where(flag, pos, torch.full_like(pos, -1))
    return pos, flag.sum(0)


class ExpertParallelMoe:
    """One MoE block spread over the ranks of `group`.  `block` is this rank's MoeBlock, built with
    its expert slice (expert_base = rank * E/N, E_local = E/N) and max_tokens >= N * n."""

    def __init__(self, block, group=None, mode: str = "all_gather", ops=None):
        if mode not in ("all_to_all", "all_gather", "a2av") and mode not in _NATIVE_MODES:
            raise ValueError("mode must be 'native', 'native_padded', 'native_exact', 'all_to_all', 'all_gather' or 'a2av'")
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
        return "native"

    def _routed_everywhere(self, x: torch.Tensor):
        """Every rank's rows, ids and weights on this rank (what the all-gather transport delivers)."""
        n = x.shape[0]
        self.block.route(x, out=(self.logits, self.w, self.idx))
        with self._batched(x.device):
            dist.all_gather_into_tensor(self.recv_x, x, group=self.group)
            dist.all_gather_into_tensor(self.recv_idx, self.idx, group=self.group)
            dist.all_gather_into_tensor(self.recv_w, self.w, group=self.group)

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
        if self.mode in _NATIVE_MODES or self.mode == "a2av":
            self._routed_everywhere(x.contiguous())
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
        if self.mode in _NATIVE_MODES:
            return self._native(x, out, stats, profile)
        if self.mode == "a2av":
            return A2avReference.forward_into(self, x, out, stats)
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

    def _native(self, x, out, stats, profile):
        """pmoe_ep_forward: route, dispatch, experts, combine behind the C ABI."""
        import ctypes as C
        from ._lib import check, lib
        from .moe import _TORCH_TO_PMOE, _check_buffer, _stream_ptr
        n, dev = x.shape[0], x.device
        _check_buffer("x", x, (n, self.H), tuple(_TORCH_TO_PMOE), dev)
        _check_buffer("out", out, (n, self.H), tuple(_TORCH_TO_PMOE), dev)
        comm = native_comm(self.group, dev)
        h = self.block._h
        if profile and not getattr(self, "_prof_on", False):
            self._call_native(h, comm, x, out, n)   # the buffers exist after the first call
            check(lib().pmoe_ep_profile(h, 1, None, None))
            self._prof_on = True
        self._mark(profile, "t0")
        self._call_native(h, comm, x, out, n)
        if stats is not None:
            stats.update(router_logits=self.logits, top_indices=self.idx, top_weights=self.w)
        if profile:
            self._mark(True, "c1")
            torch.cuda.synchronize()
            a, b = C.c_float(), C.c_float()
            check(lib().pmoe_ep_profile(h, -1, C.byref(a), C.byref(b)))
            return dict(dispatch=a.value, combine=b.value, total=self._events["t0"].elapsed_time(self._events["c1"]))
        return out

    def _call_native(self, h, comm, x, out, n):
        from ._lib import check, lib
        from .moe import _TORCH_TO_PMOE, _stream_ptr
        check(lib().pmoe_ep_forward(h, comm, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, out.data_ptr(), _TORCH_TO_PMOE[out.dtype],
                                    self.logits.data_ptr(), self.idx.data_ptr(), self.w.data_ptr(), _NATIVE_MODES[self.mode],
                                    _stream_ptr(x.device)))

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.H), dtype=out_dtype or x.dtype, device=x.device)
        return self.forward_into(x, out)


class A2avReference:
    """The native path's exchange restated with torch collectives (mode ``a2av``): the same plan, the same record order,
    the same rank-order sum -- with unquantised rows, and `block` doing the expert arithmetic.  It is what the CPU
    (gloo) test drives; on GPUs the native path is the product."""

    @staticmethod
    def forward_into(ep: "ExpertParallelMoe", x: torch.Tensor, out: torch.Tensor, stats: Optional[dict] = None):
        n, N, k, g, H = x.shape[0], ep.N, ep.k, ep.group, ep.H
        ep.block.route(x, out=(ep.logits, ep.w, ep.idx))
        if stats is not None:
            stats.update(router_logits=ep.logits, top_indices=ep.idx, top_weights=ep.w)
        pos, cnt = plan_dispatch(ep.idx, N, ep.per_rank, ep.rank, ep.round_robin, True)
        # everybody's counts: cnt_all[s][r] = records rank s sends to rank r
        cnt_all = [torch.zeros_like(cnt) for _ in range(N)]
        dist.all_gather(cnt_all, cnt, group=g)
        cnt_all = torch.stack(cnt_all)
        send_cnt = cnt_all[ep.rank].tolist()
        recv_cnt = cnt_all[:, ep.rank].tolist()
        # pack: records for rank r are the tokens with pos[:, r] >= 0, in token order; foreign ids masked
        masked = mask_for_destinations(ep.idx, N, ep.per_rank, ep.round_robin)          # [N, n, k]
        sel = [torch.nonzero(pos[:, r] >= 0).flatten() for r in range(N)]
        send_x = torch.cat([x[s] for s in sel])
        send_idx = torch.cat([masked[r][s] for r, s in enumerate(sel)])
        send_w = torch.cat([ep.w[s] for s in sel])
        rows = sum(recv_cnt)
        recv_x = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        recv_idx = torch.empty((rows, k), dtype=torch.int32, device=x.device)
        recv_w = torch.empty((rows, k), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(recv_x, send_x, recv_cnt, send_cnt, group=g)
        dist.all_to_all_single(recv_idx, send_idx, recv_cnt, send_cnt, group=g)
        dist.all_to_all_single(recv_w, send_w, recv_cnt, send_cnt, group=g)
        own_begin = sum(recv_cnt[:ep.rank])
        own = (own_begin, recv_cnt[ep.rank]) if ep.block.has_shared else None
        part = ep.block.experts_forward_batched(recv_x, recv_idx, recv_w, k, out_dtype=torch.float32, shared_rows=own)
        back = torch.empty((sum(send_cnt), H), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(back, part.contiguous(), send_cnt, recv_cnt, group=g)
        # combine: rank order
        acc = torch.zeros((n, H), dtype=torch.float32, device=x.device)
        off = 0
        for r in range(N):
            acc[sel[r]] += back[off:off + send_cnt[r]]
            off += send_cnt[r]
        out.copy_(acc)
        return out
