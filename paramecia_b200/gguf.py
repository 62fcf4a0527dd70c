"""GGUF ingestion for the MoE block: read ``blk.N.ffn_*`` tensors and the ``qwen3next.*`` metadata of
a GGUF file and hand the raw block bytes to libpmoe.

The reference loads the same tensors through candle's ``gguf_file`` reader: expert matrices
``blk.N.ffn_{gate,up,down}_exps.weight`` (paramecia-model/src/qwen3_next.rs:1256-1258), the shared
expert ``ffn_{gate,up,down}_shexp.weight`` and ``ffn_gate_inp_shexp`` (1751-1762), the router
``ffn_gate_inp.weight`` (1882) and the expert counts ``qwen3next.expert_count`` /
``qwen3next.expert_used_count`` with the ``qwen3moe.*`` fall-backs (4540-4547).  candle reverses the
GGUF dimension order, so a tensor stored with ne = [H, F, E] is the row-major [E, F, H] the
library expects; the bytes are passed on untouched.

The parser below is self-contained (GGUF v2/v3, little endian): header, key/value section, tensor
infos, aligned data section.  Tensor data is memory-mapped, nothing is converted on the host
except the small f32 vectors.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ._lib import BF16, F16, F32, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_0, row_bytes

GGUF_MAGIC = 0x46554747  # "GGUF"
DEFAULT_ALIGNMENT = 32

# GGUF metadata value types
_T_U8, _T_I8, _T_U16, _T_I16, _T_U32, _T_I32, _T_F32, _T_BOOL, _T_STR, _T_ARR, _T_U64, _T_I64, _T_F64 = range(13)
_SCALAR = {_T_U8: "<B", _T_I8: "<b", _T_U16: "<H", _T_I16: "<h", _T_U32: "<I", _T_I32: "<i", _T_F32: "<f",
           _T_BOOL: "<?", _T_U64: "<Q", _T_I64: "<q", _T_F64: "<d"}

# ggml type id -> (elements per block, bytes per block) for the types this reader can size
_GGML_SIZES = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
               2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 9: (32, 36),   # Q4_0, Q4_1, Q5_0, Q5_1, Q8_1
               10: (256, 84), 11: (256, 110), 13: (256, 176), 15: (256, 292)}     # Q2_K, Q3_K, Q5_K, Q8_K


class GGUFError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]   # row-major shape (GGUF's ne reversed), as candle reports it
    dtype: int               # ggml type id
    offset: int              # bytes from the start of the data section
    nbytes: int


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("truncated GGUF file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGUFError("truncated GGUF string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == _T_STR:
            return self.string()
        if t == _T_ARR:
            et = self.take("<I")
            n = self.take("<Q")
            if et in _SCALAR:   # bulk read
                size = struct.calcsize(_SCALAR[et])
                if self.pos + n * size > len(self.buf):
                    raise GGUFError("truncated GGUF array")
                arr = np.frombuffer(self.buf, dtype=np.dtype(_SCALAR[et][1]).newbyteorder("<"), count=n, offset=self.pos)
                self.pos += n * size
                return arr
            return [self.value(et) for _ in range(n)]
        raise GGUFError(f"unknown GGUF value type {t}")


class GGUFFile:
    """Read-only view of a GGUF file: ``metadata`` (dict), ``tensors`` (name -> TensorInfo) and
    ``tensor_bytes(name)`` (a uint8 view into the memory-mapped data section)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._mm)
        if c.take("<I") != GGUF_MAGIC:
            raise GGUFError(f"{path}: not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GGUFError(f"{path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors = c.take("<Q")
        n_kv = c.take("<Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.take("<I"))
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            ne = [c.take("<Q") for _ in range(nd)]
            dtype = c.take("<I")
            offset = c.take("<Q")
            if dtype not in _GGML_SIZES:
                nbytes = -1   # a type this reader cannot size; only an error if the tensor is asked for
            else:
                be, bb = _GGML_SIZES[dtype]
                n = int(np.prod(ne, dtype=np.int64)) if ne else 1
                if ne and ne[0] % be:
                    raise GGUFError(f"{name}: first dimension {ne[0]} is not a multiple of the block size {be}")
                nbytes = n // be * bb
            self.tensors[name] = TensorInfo(name, tuple(reversed(ne)), dtype, offset, nbytes)
        align = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (c.pos + align - 1) // align * align

    def close(self):
        if self._mm is not None:
            self._mm.close()
            self._f.close()
            self._mm = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def meta(self, *keys, default=None):
        """First of `keys` that is present (the reference tries ``qwen3next.*`` then ``qwen3moe.*``)."""
        for k in keys:
            if k in self.metadata:
                return self.metadata[k]
        return default

    def tensor_bytes(self, name: str) -> np.ndarray:
        t = self.tensors.get(name)
        if t is None:
            raise GGUFError(f"{self.path}: no tensor named {name}")
        if t.nbytes < 0:
            raise GGUFError(f"{name}: ggml type {t.dtype} is not supported")
        lo = self.data_start + t.offset
        if lo + t.nbytes > len(self._mm):
            raise GGUFError(f"{name}: data runs past the end of the file")
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=lo)


# ---------------------------------------------------------------------------------------------
# MoE block from a GGUF file

def _host_tensor(view: np.ndarray) -> torch.Tensor:
    """uint8 torch tensor over a read-only memory-mapped view, without a host copy."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)   # "buffer is not writable": it is only read
        return torch.from_numpy(view)


def _float_tensor(f: GGUFFile, name: str, device, keep_16bit: bool = False) -> torch.Tensor:
    """A float tensor of the file as torch f32 (or, with keep_16bit, in its own 16-bit type).
    Quantised tensors are dequantised by the library's bit-exact codec (QTensor::dequantize)."""
    t = f.tensors[name]
    raw = _host_tensor(f.tensor_bytes(name))
    if t.dtype == F32:
        return raw.view(torch.float32).reshape(t.shape).to(device)
    if t.dtype in (F16, BF16):
        v = raw.view(torch.float16 if t.dtype == F16 else torch.bfloat16).reshape(t.shape).to(device)
        return v if keep_16bit else v.float()
    if t.dtype in (Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K):
        from .moe import dequantize
        n = int(np.prod(t.shape))
        return dequantize(raw.to(device), t.dtype, n).reshape(t.shape)
    raise GGUFError(f"{name}: ggml type {t.dtype} cannot be read as floats here")


def moe_layer_names(layer: int) -> Dict[str, str]:
    p = f"blk.{layer}"
    return dict(gate_exps=f"{p}.ffn_gate_exps.weight", up_exps=f"{p}.ffn_up_exps.weight",
                down_exps=f"{p}.ffn_down_exps.weight", router=f"{p}.ffn_gate_inp.weight",
                sh_gate=f"{p}.ffn_gate_shexp.weight", sh_up=f"{p}.ffn_up_shexp.weight",
                sh_down=f"{p}.ffn_down_shexp.weight", sh_gate_inp=f"{p}.ffn_gate_inp_shexp.weight",
                sh_gate_inp_alt=f"{p}.ffn_gate_inp_shexp")


def moe_layers(f: GGUFFile):
    """Indices of the layers that hold a sparse MoE FFN (have ``ffn_gate_exps``)."""
    out = []
    for name in f.tensors:
        parts = name.split(".")
        if len(parts) == 4 and parts[0] == "blk" and parts[2] == "ffn_gate_exps" and parts[3] == "weight":
            out.append(int(parts[1]))
    return sorted(out)


def load_moe_block(f: GGUFFile, layer: int, device="cuda:0", max_tokens: int = 256, ep_rank: int = 0,
                   ep_size: int = 1, num_experts_per_tok: Optional[int] = None):
    """MoeBlock::new for ``blk.<layer>`` of an open GGUF file (qwen3_next.rs:1853-1896): the raw
    blocks of the expert tensors go to the device as they are; with ep_size > 1 only this rank's
    contiguous slice of the experts is read."""
    from .moe import MoeBlock, QTensor, SharedExpertWeights
    names = moe_layer_names(layer)
    for k in ("gate_exps", "up_exps", "down_exps", "router"):
        if names[k] not in f.tensors:
            raise GGUFError(f"{f.path}: layer {layer} has no {names[k]}")
    g, u, d = (f.tensors[names[k]] for k in ("gate_exps", "up_exps", "down_exps"))
    if len(g.shape) != 3 or g.shape != u.shape or d.shape != (g.shape[0], g.shape[2], g.shape[1]):
        raise GGUFError(f"layer {layer}: expert tensors have shapes {g.shape}, {u.shape}, {d.shape}; "
                        "expected [E,F,H], [E,F,H], [E,H,F]")
    E, F, H = g.shape   # the reference takes the expert count from the tensor shape (qwen3_next.rs:1262)
    if E % ep_size:
        raise GGUFError(f"{E} experts do not divide over {ep_size} ranks")
    El = E // ep_size
    base = ep_rank * El
    k = num_experts_per_tok or int(f.meta("qwen3next.expert_used_count", "qwen3moe.expert_used_count", default=8))

    def experts(info: TensorInfo, rows: int, cols: int) -> QTensor:
        per = rows * row_bytes(info.dtype, cols)
        if per <= 0:
            raise GGUFError(f"{info.name}: ggml type {info.dtype} is not an expert type this library serves")
        raw = f.tensor_bytes(info.name)[base * per:(base + El) * per]
        return QTensor(_host_tensor(raw).to(device), info.dtype, (El, rows, cols))

    router_info = f.tensors[names["router"]]
    if router_info.shape != (E, H):
        raise GGUFError(f"{router_info.name}: shape {router_info.shape}, expected {(E, H)}")
    if router_info.dtype in (F32, F16, BF16):
        router = _float_tensor(f, names["router"], device, keep_16bit=True)
    else:
        # a quantised router is a quantised mat-mul in the reference (Q8 activations, integer block dots); the
        # library runs it that way, so the blocks go over as they are
        if row_bytes(router_info.dtype, H) <= 0:
            raise GGUFError(f"{router_info.name}: ggml type {router_info.dtype} is not a type this library serves")
        router = QTensor(_host_tensor(f.tensor_bytes(router_info.name)).to(device), router_info.dtype, (E, H))

    shared = None
    if names["sh_up"] in f.tensors:   # SharedExpert::new returns None without ffn_up_shexp (qwen3_next.rs:1751-1754)
        gi = names["sh_gate_inp"] if names["sh_gate_inp"] in f.tensors else names["sh_gate_inp_alt"]
        if gi not in f.tensors:
            raise GGUFError(f"layer {layer}: shared expert without ffn_gate_inp_shexp")

        def mat(key: str, rows: int, cols: int) -> QTensor:
            info = f.tensors[names[key]]
            if info.shape != (rows, cols):
                raise GGUFError(f"{info.name}: shape {info.shape}, expected {(rows, cols)}")
            return QTensor(_host_tensor(f.tensor_bytes(info.name)).to(device), info.dtype, (rows, cols))

        gate_vec = _float_tensor(f, gi, device).reshape(-1)
        if gate_vec.numel() != H:
            raise GGUFError(f"{gi}: {gate_vec.numel()} elements, expected {H}")
        shared = SharedExpertWeights(mat("sh_gate", F, H), mat("sh_up", F, H), mat("sh_down", H, F), gate_vec)

    return MoeBlock(experts(g, F, H), experts(u, F, H), experts(d, H, F), router, k, shared_expert=shared, device=device,
                    max_tokens=max_tokens, num_experts=E, expert_base=base)
