"""Host-side mirror of the reference's MoE block interface over libpmoe.

Names and argument meaning follow paramecia-model/src/qwen3_next.rs:

* ``QTensor``            -- candle's quantised tensor as the reference uses it: raw GGUF blocks,
                            a GGML dtype and a shape; ``dequantize`` is QTensor::dequantize.
* ``MoeBlock``           -- MoeBlock (1840-2218): ``forward`` / ``forward_with_stats`` return what
                            the Rust methods return; ``top_k`` is ops::topk_moe_routing on the
                            block's own router; ``experts_forward_batched`` is
                            MoeExperts::forward_batched (1347-1394); ``shared_forward`` is
                            SharedExpert::forward (1776-1823).

Tensors are torch CUDA tensors; this module only checks shapes, allocates outputs and passes
raw pointers and the current stream to the C ABI.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import BF16, F16, F32, LayerDesc, PmoeError, check, lib, row_bytes

_TORCH_TO_PMOE = {torch.float32: F32, torch.bfloat16: BF16}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _as_u8(data, device=None) -> torch.Tensor:
    if isinstance(data, np.ndarray):
        data = torch.from_numpy(np.ascontiguousarray(data).view(np.uint8).reshape(-1))
    if data.dtype != torch.uint8:
        data = data.contiguous().view(torch.uint8)
    data = data.reshape(-1).contiguous()
    if device is not None:
        data = data.to(device)
    return data


class QTensor:
    """Raw GGUF blocks with a GGML dtype id and a logical shape (rows..., cols)."""

    def __init__(self, data, dtype: int, shape: Tuple[int, ...]):
        self.data = _as_u8(data)
        self.dtype = int(dtype)
        self.shape = tuple(int(s) for s in shape)
        n = 1
        for s in self.shape:
            n *= s
        expect = n // _lib.block_size(self.dtype) * _lib.type_size(self.dtype)
        if self.data.numel() != expect:
            raise ValueError(f"QTensor: {self.data.numel()} bytes given, shape {self.shape} needs {expect}")

    @property
    def device(self):
        return self.data.device

    def to(self, device) -> "QTensor":
        return QTensor(self.data.to(device), self.dtype, self.shape)

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def slice_first_dim(self, index: int) -> "QTensor":
        """QTensor::slice_first_dim: expert `index` is one contiguous byte range."""
        per = self.data.numel() // self.shape[0]
        return QTensor(self.data[index * per:(index + 1) * per], self.dtype, self.shape[1:])

    def dequantize(self, device=None) -> torch.Tensor:
        dev = torch.device(device) if device is not None else self.data.device
        return dequantize(self.data.to(dev), self.dtype, self.numel()).reshape(self.shape)


def dequantize(blocks: torch.Tensor, dtype: int, n_elems: int) -> torch.Tensor:
    """QTensor::dequantize on the GPU: raw blocks (uint8, CUDA) -> f32."""
    if not blocks.is_cuda:
        raise PmoeError(-9, "dequantize needs CUDA tensors; libpmoe has no CPU path")
    blocks = blocks.contiguous()
    out = torch.empty(n_elems, dtype=torch.float32, device=blocks.device)
    check(lib().pmoe_dequantize(blocks.device.index or 0, dtype, blocks.data_ptr(), n_elems, out.data_ptr(),
                                _stream_ptr(blocks.device)))
    return out


def qmatmul(w: "QTensor", x: torch.Tensor) -> torch.Tensor:
    """QMatMul::forward for a quantised [rows, cols] tensor: x [m, cols] f32 -> [m, rows] f32."""
    rows, cols = w.shape
    x = x.to(torch.float32).reshape(-1, cols).contiguous()
    data = w.data.to(x.device)
    y = torch.empty((x.shape[0], rows), dtype=torch.float32, device=x.device)
    check(lib().pmoe_qmatmul(x.device.index or 0, w.dtype, data.data_ptr(), rows, cols, x.data_ptr(), x.shape[0],
                             y.data_ptr(), _stream_ptr(x.device)))
    return y


def modify_block_scales(w: "QTensor", mults: torch.Tensor) -> "QTensor":
    """QTensor::modify_block_scales: a new QTensor whose block i carries its f16 scale(s) times mults[i]."""
    if not w.data.is_cuda:
        raise PmoeError(-9, "modify_block_scales needs CUDA tensors; libpmoe has no CPU path")
    n_blocks = w.numel() // _lib.block_size(w.dtype)
    m = mults.to(w.data.device, torch.float32).reshape(-1).contiguous()
    if m.numel() != n_blocks:
        raise ValueError(f"{m.numel()} multipliers given, the tensor has {n_blocks} blocks")
    out = torch.empty_like(w.data)
    check(lib().pmoe_modify_block_scales(w.data.device.index or 0, w.dtype, w.data.data_ptr(), n_blocks, m.data_ptr(),
                                         out.data_ptr(), _stream_ptr(w.data.device)))
    return QTensor(out, w.dtype, w.shape)


def qmatmul_noalloc(w: "QTensor", x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """`qmatmul` through the entry point that allocates nothing: the caller owns x [m, cols] f32 and
    y [m, rows] f32 (both CUDA, contiguous) and the quantised activations use the library's built-in
    96 KB buffer, so m * cols <= 78 028 (38 rows of 2048 columns).  Calls on one device must not overlap."""
    rows, cols = w.shape
    if not w.data.is_cuda:
        raise ValueError("qmatmul_noalloc takes CUDA tensors it does not have to copy")
    if x.dim() != 2:
        raise ValueError("x must be [m, cols]")
    _check_buffer("x", x, (x.shape[0], cols), torch.float32, w.data.device)
    _check_buffer("y", y, (x.shape[0], rows), torch.float32, w.data.device)
    check(lib().pmoe_qmatmul_noalloc(x.device.index or 0, w.dtype, w.data.data_ptr(), rows, cols, x.data_ptr(),
                                     x.shape[0], y.data_ptr(), _stream_ptr(x.device)))
    return y


def add_rms_norm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                 eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(resid + delta, RmsNorm(resid + delta)): quantized_nn.rs:172-190 with the residual add
    of LayerWeights::forward_with_stats (qwen3_next.rs:4273-4286)."""
    n, H = resid.shape
    resid = resid.contiguous()
    new_resid = torch.empty_like(resid)
    y = torch.empty_like(resid)
    check(lib().pmoe_add_rms_norm(resid.device.index or 0, resid.data_ptr(),
                                  None if delta is None else delta.contiguous().data_ptr(),
                                  None if weight is None else weight.contiguous().data_ptr(),
                                  n, H, float(eps), new_resid.data_ptr(), y.data_ptr(), _stream_ptr(resid.device)))
    return new_resid, y


def add_rms_norm_into(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                      resid_out: torch.Tensor, y: torch.Tensor) -> None:
    """`add_rms_norm` into caller-owned f32 [n, H] buffers (nothing is allocated); `resid_out` may be `resid`."""
    n, H = resid.shape
    for name, t in (("resid", resid), ("resid_out", resid_out), ("y", y)) + ((("delta", delta),) if delta is not None else ()):
        _check_buffer(name, t, (n, H), torch.float32, resid.device)
    if weight is not None:
        _check_buffer("weight", weight, (H,), torch.float32, resid.device)
    check(lib().pmoe_add_rms_norm(resid.device.index or 0, resid.data_ptr(),
                                  None if delta is None else delta.data_ptr(),
                                  None if weight is None else weight.data_ptr(),
                                  n, H, float(eps), resid_out.data_ptr(), y.data_ptr(), _stream_ptr(resid.device)))


def _check_buffer(name: str, t: torch.Tensor, shape, dtype, device) -> None:
    """A caller-owned buffer whose raw pointer goes to the C ABI: the library cannot see its size or type, so a wrong
    one would be read or written out of bounds on the device.  Refuse it here."""
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a torch tensor")
    if t.device != torch.device(device):
        raise ValueError(f"{name} must live on {device} (got {t.device})")
    dtypes = dtype if isinstance(dtype, (tuple, list)) else (dtype,)
    if t.dtype not in dtypes:
        raise ValueError(f"{name} must be {' or '.join(str(d) for d in dtypes)} (got {t.dtype})")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)} (got {tuple(t.shape)})")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


@dataclass
class SharedExpertWeights:
    """ffn_{gate,up,down}_shexp.weight and ffn_gate_inp_shexp (qwen3_next.rs:1749-1774)."""
    gate_proj: QTensor   # [F, H]
    up_proj: QTensor     # [F, H]
    down_proj: QTensor   # [H, F]
    shared_gate: torch.Tensor  # [H] f32


class MoeBlock:
    """One Qwen3-Next sparse MoE FFN block resident on one GPU.

    gate_exps / up_exps: QTensor [E_local, F, H]; down_exps: QTensor [E_local, H, F];
    gate (router): f32 / f16 / bf16 tensor [E, H], or a QTensor [E, H] (quantised router).  With expert parallelism a rank passes its slice of the
    experts and ``expert_base``; indices outside the slice contribute nothing.
    """

    def __init__(self, gate_exps: QTensor, up_exps: QTensor, down_exps: QTensor, gate: torch.Tensor,
                 num_experts_per_tok: int, shared_expert: Optional[SharedExpertWeights] = None,
                 device="cuda:0", max_tokens: int = 256, router_bias: Optional[torch.Tensor] = None,
                 num_experts: Optional[int] = None, expert_base: int = 0, training_mode: bool = False,
                 ep_rank: int = 0, ep_size: int = 0, ep_placement: str = "contiguous"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise PmoeError(-9, "MoeBlock needs a CUDA device; libpmoe has no CPU path")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        E_local, F, H = gate_exps.shape
        self.hidden_dim, self.n_ff = H, F
        self.num_experts = int(num_experts) if num_experts is not None else int(gate.shape[0])
        self.num_experts_local = E_local
        self.expert_base = int(expert_base)
        if ep_placement not in ("contiguous", "round_robin"):
            raise ValueError("ep_placement must be 'contiguous' or 'round_robin'")
        self.ep_placement = 1 if ep_placement == "round_robin" else 0
        self.ep_rank, self.ep_size = int(ep_rank), int(ep_size)
        self.num_experts_per_tok = int(num_experts_per_tok)
        self.max_tokens = int(max_tokens)
        if tuple(up_exps.shape) != (E_local, F, H) or tuple(down_exps.shape) != (E_local, H, F):
            raise ValueError("expert tensor shapes must be [E,F,H], [E,F,H], [E,H,F]")
        if tuple(gate.shape) != (self.num_experts, H):
            raise ValueError("router weight must be [E, H]")
        if isinstance(gate, QTensor):
            # a quantised ffn_gate_inp: the library runs it as a quantised mat-mul, like the reference's QMatMul
            router_dt, router = int(gate.dtype), gate.data.to(self.device).contiguous()
        else:
            # f16 / bf16 router weights go to the library as they are (it widens them once); others as f32
            router_dt = {torch.float16: F16, torch.bfloat16: BF16}.get(gate.dtype, F32)
            router = gate.to(self.device).contiguous() if router_dt != F32 else gate.to(self.device, torch.float32).contiguous()
        # the library adopts these device buffers in place (weights_location = 2); keep them alive
        self._keep = dict(
            gate=gate_exps.data.to(self.device), up=up_exps.data.to(self.device),
            down=down_exps.data.to(self.device),
            router=router,
            bias=None if router_bias is None else router_bias.to(self.device, torch.float32).contiguous())
        d = LayerDesc()
        d.struct_size = C.sizeof(LayerDesc)
        d.device = self.device.index
        d.H, d.F, d.E, d.k = H, F, self.num_experts, self.num_experts_per_tok
        d.max_tokens = self.max_tokens
        d.expert_base, d.E_local = self.expert_base, E_local
        d.gate_dtype, d.up_dtype, d.down_dtype = gate_exps.dtype, up_exps.dtype, down_exps.dtype
        d.gate_exps, d.up_exps, d.down_exps = (self._keep[k].data_ptr() for k in ("gate", "up", "down"))
        d.has_shared = 0
        if shared_expert is not None:
            s = shared_expert
            self._keep.update(sg=s.gate_proj.data.to(self.device), su=s.up_proj.data.to(self.device),
                              sd=s.down_proj.data.to(self.device),
                              sgi=s.shared_gate.to(self.device, torch.float32).contiguous())
            d.has_shared = 1
            d.sh_gate_dtype, d.sh_up_dtype, d.sh_down_dtype = s.gate_proj.dtype, s.up_proj.dtype, s.down_proj.dtype
            d.sh_gate, d.sh_up, d.sh_down = (self._keep[k].data_ptr() for k in ("sg", "su", "sd"))
            d.sh_gate_inp = self._keep["sgi"].data_ptr()
        d.router_dtype = router_dt
        d.router_w = self._keep["router"].data_ptr()
        d.router_bias = None if self._keep["bias"] is None else self._keep["bias"].data_ptr()
        d.weights_location = 2
        d.training_mode = 1 if training_mode else 0
        d.ep_placement, d.ep_rank, d.ep_size = self.ep_placement, self.ep_rank, self.ep_size
        self.has_shared = shared_expert is not None
        self._desc = d
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().pmoe_layer_create(C.byref(d), C.byref(self._h)))

    # -- lifetime -------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            lib().pmoe_layer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers --------------------------------------------------------------------
    def _flat(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.dtype not in _TORCH_TO_PMOE:
            raise PmoeError(-2, f"activations must be float32 or bfloat16, got {hidden_states.dtype}")
        if not hidden_states.is_cuda:
            raise PmoeError(-9, "activations must be CUDA tensors; use forward_host for host buffers")
        if hidden_states.shape[-1] != self.hidden_dim:
            raise ValueError(f"last dim must be {self.hidden_dim}")
        return hidden_states.reshape(-1, self.hidden_dim).contiguous()

    def local_mask(self, idx: torch.Tensor) -> torch.Tensor:
        """Which entries of a routing table name an expert this handle holds."""
        idx = idx.to(torch.int64)
        if self.ep_placement == 1:
            return (idx >= 0) & (idx < self.num_experts) & (idx % self.ep_size == self.ep_rank)
        return (idx >= self.expert_base) & (idx < self.expert_base + self.num_experts_local)

    def resident_bytes(self) -> int:
        """Bytes of weights this handle keeps in HBM."""
        return int(sum(v.numel() * v.element_size() for v in self._keep.values() if v is not None))

    def weight_bytes(self, distinct_experts: int) -> int:
        """Algorithmic weight bytes one decode call streams when `distinct_experts` experts are hit."""
        d = self._desc
        per = self.n_ff * (row_bytes(d.gate_dtype, d.H) + row_bytes(d.up_dtype, d.H)) + d.H * row_bytes(d.down_dtype, d.F)
        b = distinct_experts * per + self.num_experts * d.H * 4
        if self.has_shared:
            b += self.n_ff * (row_bytes(d.sh_gate_dtype, d.H) + row_bytes(d.sh_up_dtype, d.H)) \
                + d.H * row_bytes(d.sh_down_dtype, d.F)
        return b

    # -- the reference's methods ----------------------------------------------------
    def forward_with_stats(self, hidden_states: torch.Tensor, out_dtype: Optional[torch.dtype] = None):
        """MoeBlock::forward_with_stats: ``(out [b,l,H], (router_logits [b,l,E], top_indices [b,l,k]))``.
        The logits are the unclamped ones; indices are int32 tensors holding the u32 ids."""
        shape = hidden_states.shape
        x = self._flat(hidden_states)
        n = x.shape[0]
        out_dtype = out_dtype or hidden_states.dtype
        out = torch.empty((n, self.hidden_dim), dtype=out_dtype, device=self.device)
        logits = torch.empty((n, self.num_experts), dtype=torch.float32, device=self.device)
        idx = torch.empty((n, self.num_experts_per_tok), dtype=torch.int32, device=self.device)
        w = torch.empty((n, self.num_experts_per_tok), dtype=torch.float32, device=self.device)
        check(lib().pmoe_forward(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, out.data_ptr(),
                                 _TORCH_TO_PMOE[out_dtype], logits.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                 _stream_ptr(self.device)))
        self.last_top_weights = w
        lead = tuple(shape[:-1])
        return out.reshape(*lead, self.hidden_dim), (logits.reshape(*lead, self.num_experts),
                                                     idx.reshape(*lead, self.num_experts_per_tok))

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """MoeBlock::forward."""
        return self.forward_with_stats(hidden_states)[0]

    def forward_into(self, x: torch.Tensor, out: torch.Tensor):
        """forward with caller-owned buffers and no stats (nothing is allocated; graph-capturable)."""
        if x.dim() != 2 or x.shape[1] != self.hidden_dim:
            raise ValueError(f"x must be [n, {self.hidden_dim}]")
        n = x.shape[0]
        _check_buffer("x", x, (n, self.hidden_dim), tuple(_TORCH_TO_PMOE), self.device)
        _check_buffer("out", out, (n, self.hidden_dim), tuple(_TORCH_TO_PMOE), self.device)
        check(lib().pmoe_forward(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, out.data_ptr(),
                                 _TORCH_TO_PMOE[out.dtype], None, None, None, _stream_ptr(self.device)))

    def route(self, hidden_states: torch.Tensor, out=None):
        """gate.forward -> clamp -> softmax -> top_k: ``(router_logits, top_weights, top_indices)``.
        `out` = the three result tensors to fill (f32 [n,E], f32 [n,k], int32 [n,k], contiguous)."""
        x = self._flat(hidden_states)
        n = x.shape[0]
        if out is not None:
            logits, w, idx = out
            _check_buffer("router_logits", logits, (n, self.num_experts), torch.float32, self.device)
            _check_buffer("top_weights", w, (n, self.num_experts_per_tok), torch.float32, self.device)
            _check_buffer("top_indices", idx, (n, self.num_experts_per_tok), torch.int32, self.device)
        else:
            logits = torch.empty((n, self.num_experts), dtype=torch.float32, device=self.device)
            idx = torch.empty((n, self.num_experts_per_tok), dtype=torch.int32, device=self.device)
            w = torch.empty((n, self.num_experts_per_tok), dtype=torch.float32, device=self.device)
        check(lib().pmoe_route(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, logits.data_ptr(), idx.data_ptr(),
                               w.data_ptr(), _stream_ptr(self.device)))
        return logits, w, idx

    def router_stats(self, router_logits: torch.Tensor, top_indices: torch.Tensor):
        """Per-block pieces of compute_z_loss / compute_load_balance_loss (qwen3_next.rs:5549-5648):
        ``(expert_counts [E] f32, z_loss, load_balance_loss)`` as device tensors, unweighted."""
        E = self.num_experts
        logits = router_logits.to(self.device, torch.float32).reshape(-1, E).contiguous()
        n = logits.shape[0]
        idx = top_indices.to(self.device, torch.int32).reshape(n, -1).contiguous()
        counts = torch.zeros(E, dtype=torch.float32, device=self.device)
        losses = torch.zeros(2, dtype=torch.float32, device=self.device)
        check(lib().pmoe_router_stats(self._h, logits.data_ptr(), idx.data_ptr(), n, idx.shape[1], counts.data_ptr(),
                                      losses.data_ptr(), _stream_ptr(self.device)))
        return counts, losses[0], losses[1]

    def experts_forward_batched(self, hidden_states: torch.Tensor, expert_indices: torch.Tensor,
                                expert_weights: torch.Tensor, top_k: Optional[int] = None,
                                out_dtype: Optional[torch.dtype] = None,
                                shared_rows: Optional[Tuple[int, int]] = None,
                                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """MoeExperts::forward_batched(hidden [n,H], indices [n,k] u32, weights [n,k] f32, top_k).

        shared_rows = (begin, count) adds the shared expert on those rows in the same kernels
        (the expert-parallel form: a rank passes the range of its own tokens); `out` = the
        contiguous [n, H] tensor to fill."""
        x = self._flat(hidden_states)
        n = x.shape[0]
        top_k = int(top_k or expert_indices.shape[-1])
        idx = expert_indices.to(self.device, torch.int32).reshape(n, top_k).contiguous()
        w = expert_weights.to(self.device, torch.float32).reshape(n, top_k).contiguous()
        if out is None:
            out_dtype = out_dtype or hidden_states.dtype
            out = torch.empty((n, self.hidden_dim), dtype=out_dtype, device=self.device)
        else:
            _check_buffer("out", out, (n, self.hidden_dim), tuple(_TORCH_TO_PMOE), self.device)
            out_dtype = out.dtype
        if shared_rows is not None:
            check(lib().pmoe_experts_forward_ep(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], idx.data_ptr(),
                                                w.data_ptr(), n, top_k, int(shared_rows[0]), int(shared_rows[1]),
                                                out.data_ptr(), _TORCH_TO_PMOE[out_dtype], _stream_ptr(self.device)))
            return out
        check(lib().pmoe_experts_forward(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], idx.data_ptr(), w.data_ptr(),
                                         n, top_k, out.data_ptr(), _TORCH_TO_PMOE[out_dtype], _stream_ptr(self.device)))
        return out

    def _blocks_of(self, which: str) -> int:
        d = self._desc
        El, F, H = self.num_experts_local, self.n_ff, self.hidden_dim
        return {"gate": El * F * (H // _lib.block_size(d.gate_dtype)), "up": El * F * (H // _lib.block_size(d.up_dtype)),
                "down": El * H * (F // _lib.block_size(d.down_dtype)),
                "sh_gate": F * (H // max(1, _lib.block_size(d.sh_gate_dtype))), "sh_up": F * (H // max(1, _lib.block_size(d.sh_up_dtype))),
                "sh_down": H * (F // max(1, _lib.block_size(d.sh_down_dtype)))}[which]

    def _mults(self, name: str, which: str, m: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if m is None:
            return None
        m = m.to(self.device, torch.float32).reshape(-1).contiguous()
        if m.numel() != self._blocks_of(which):
            raise ValueError(f"{name}: {m.numel()} multipliers given, the tensor has {self._blocks_of(which)} blocks")
        return m

    def set_block_multipliers(self, gate_mults: torch.Tensor, up_mults: torch.Tensor, down_mults: torch.Tensor) -> None:
        """MoeExperts::set_block_multipliers (qwen3_next.rs:1705-1720): one f32 multiplier per quantisation block
        of this handle's gate / up / down expert tensors, in storage order.  Every later forward uses the scaled
        weights (QTensor::modify_block_scales, build_scaled_mats 1554-1621) on the fast paths."""
        g, u, d = (self._mults(n, w, m) for n, w, m in (("gate_mults", "gate", gate_mults), ("up_mults", "up", up_mults),
                                                          ("down_mults", "down", down_mults)))
        check(lib().pmoe_layer_set_block_multipliers(self._h, g.data_ptr(), u.data_ptr(), d.data_ptr(), _stream_ptr(self.device)))

    def clear_block_multipliers(self) -> None:
        """MoeExperts::clear_block_multipliers (qwen3_next.rs:1722-1732)."""
        check(lib().pmoe_layer_set_block_multipliers(self._h, None, None, None, _stream_ptr(self.device)))

    def set_shared_scales(self, gate_scales: Optional[torch.Tensor] = None, up_scales: Optional[torch.Tensor] = None,
                          down_scales: Optional[torch.Tensor] = None) -> None:
        """SharedExpert's custom_gate_scales / custom_up_scales / custom_down_scales (qwen3_next.rs:1743-1745,
        1780-1799); None leaves that matrix unscaled."""
        g, u, d = (self._mults(n, w, m) for n, w, m in (("gate_scales", "sh_gate", gate_scales), ("up_scales", "sh_up", up_scales),
                                                          ("down_scales", "sh_down", down_scales)))
        check(lib().pmoe_layer_set_shared_scales(self._h, *(None if t is None else t.data_ptr() for t in (g, u, d)),
                                                 _stream_ptr(self.device)))

    def shared_forward(self, hidden_states: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """SharedExpert::forward, sigmoid gate included."""
        shape = hidden_states.shape
        x = self._flat(hidden_states)
        n = x.shape[0]
        out_dtype = out_dtype or hidden_states.dtype
        out = torch.empty((n, self.hidden_dim), dtype=out_dtype, device=self.device)
        check(lib().pmoe_shared_forward(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, out.data_ptr(),
                                        _TORCH_TO_PMOE[out_dtype], _stream_ptr(self.device)))
        return out.reshape(shape)

    def forward_host(self, x_host: torch.Tensor, out_host: Optional[torch.Tensor] = None, with_stats: bool = False):
        """The block with HOST tensors: host->device copy, kernels, device->host copy, synchronised."""
        if x_host.is_cuda:
            raise ValueError("forward_host takes host tensors")
        x = x_host.reshape(-1, self.hidden_dim).contiguous()
        n = x.shape[0]
        if out_host is None:
            out_host = torch.empty((n, self.hidden_dim), dtype=x.dtype)
        logits = idx = w = None
        if with_stats:
            logits = torch.empty((n, self.num_experts), dtype=torch.float32)
            idx = torch.empty((n, self.num_experts_per_tok), dtype=torch.int32)
            w = torch.empty((n, self.num_experts_per_tok), dtype=torch.float32)
        check(lib().pmoe_forward_host(self._h, x.data_ptr(), _TORCH_TO_PMOE[x.dtype], n, out_host.data_ptr(),
                                      _TORCH_TO_PMOE[out_host.dtype],
                                      None if logits is None else logits.data_ptr(),
                                      None if idx is None else idx.data_ptr(),
                                      None if w is None else w.data_ptr(), _stream_ptr(self.device)))
        return (out_host, (logits, idx, w)) if with_stats else out_host

    def trace(self, enable: bool = True):
        """Turns per-phase CUDA-event timing of forward calls on or off."""
        check(lib().pmoe_layer_trace(self._h, 1 if enable else 0))

    def trace_read(self):
        """Milliseconds per phase of the last traced forward call: {phase name: ms}."""
        ms = (C.c_float * _lib.TRACE_PHASES)()
        check(lib().pmoe_layer_trace_read(self._h, ms))
        return {lib().pmoe_trace_phase_name(i).decode(): float(ms[i]) for i in range(_lib.TRACE_PHASES)}

    def status(self):
        """Synchronises and raises PmoeError if a kernel recorded a timeout or a bad index."""
        check(lib().pmoe_layer_status(self._h, _stream_ptr(self.device)))
