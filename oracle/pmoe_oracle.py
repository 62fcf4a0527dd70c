"""ctypes binding of the CPU oracle (``libpmoe_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.  The product package never imports it.

PARITY UNPINNED against the Rust reference (it cannot be built here and carries no golden
vectors for this path); the block codecs are pinned against gguf-py in ``tests/golden``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpmoe_oracle.so")

F32, F16, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 0, 1, 8, 10, 11, 12, 13, 14
DTYPE_NAMES = {F32: "F32", F16: "F16", Q8_0: "Q8_0", Q2_K: "Q2_K", Q3_K: "Q3_K", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the shared object is missing or stale."""
    src = os.path.join(_HERE, "pmoe_oracle.c")
    hdr = os.path.join(_HERE, "pmoe_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libpmoe_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


class _Layer(C.Structure):
    _fields_ = [
        ("H", C.c_int32), ("F", C.c_int32), ("E", C.c_int32), ("k", C.c_int32),
        ("gate_dtype", C.c_int32), ("up_dtype", C.c_int32), ("down_dtype", C.c_int32),
        ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
        ("has_shared", C.c_int32),
        ("sh_gate_dtype", C.c_int32), ("sh_up_dtype", C.c_int32), ("sh_down_dtype", C.c_int32),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
        ("sh_gate_inp", C.c_void_p), ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
        ("router_dtype", C.c_int32), ("router_q", C.c_void_p),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.pmo_block_size.restype = C.c_size_t
        L.pmo_type_size.restype = C.c_size_t
        L.pmo_row_bytes.restype = C.c_size_t
        L.pmo_row_bytes.argtypes = [C.c_int, C.c_size_t]
        L.pmo_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.pmo_quantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.pmo_modify_block_scales.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
        L.pmo_quantize_q8k.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
        L.pmo_quantize_q8k.restype = None
        L.pmo_quantize_q8_0_act.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
        L.pmo_quantize_q8_0_act.restype = None
        L.pmo_qmatmul.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]
        L.pmo_router_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        L.pmo_router_logits.restype = None
        L.pmo_layer_router_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.pmo_layer_router_logits.restype = C.c_int
        L.pmo_route_topk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.pmo_route_topk.restype = None
        L.pmo_experts_forward.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.pmo_shared_forward.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_int, C.c_void_p]
        L.pmo_moe_forward.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.pmo_moe_forward_exact.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.pmo_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p]
        L.pmo_rms_norm.restype = None
        L.pmo_set_threads.argtypes = [C.c_int]
        L.pmo_set_threads.restype = None
        L.pmo_simd_kind.restype = C.c_char_p
        L.pmo_set_simd.argtypes = [C.c_int]
        L.pmo_set_simd.restype = None
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def block_size(dtype): return lib().pmo_block_size(dtype)
def type_size(dtype): return lib().pmo_type_size(dtype)
def row_bytes(dtype, cols): return lib().pmo_row_bytes(dtype, cols)
def max_threads(): return lib().pmo_max_threads()
def set_threads(n): lib().pmo_set_threads(int(n))
def simd_kind(): return lib().pmo_simd_kind().decode()
def set_simd(on): lib().pmo_set_simd(1 if on else 0)


def dequantize(dtype: int, blocks: np.ndarray, n_elems: int) -> np.ndarray:
    blocks = _c(blocks, np.uint8)
    out = np.empty(n_elems, np.float32)
    if lib().pmo_dequantize(dtype, _p(blocks), n_elems, _p(out)):
        raise ValueError("pmo_dequantize failed")
    return out


def quantize(dtype: int, x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32).ravel()
    nbytes = x.size // block_size(dtype) * type_size(dtype)
    out = np.empty(nbytes, np.uint8)
    if lib().pmo_quantize(dtype, _p(x), x.size, _p(out)):
        raise ValueError("pmo_quantize failed")
    return out


def modify_block_scales(dtype: int, blocks: np.ndarray, mults: np.ndarray) -> np.ndarray:
    """QTensor::modify_block_scales: a copy of `blocks` whose block i has its f16 scale(s) times mults[i]."""
    blocks = _c(blocks, np.uint8).ravel()
    mults = _c(mults, np.float32).ravel()
    if blocks.size != mults.size * type_size(dtype):
        raise ValueError("one multiplier per block")
    out = np.empty_like(blocks)
    if lib().pmo_modify_block_scales(dtype, _p(blocks), mults.size, _p(mults), _p(out)):
        raise ValueError("pmo_modify_block_scales failed")
    return out


def quantize_q8k(x: np.ndarray):
    x = _c(x, np.float32).ravel()
    nb = x.size // 256
    d = np.empty(nb, np.float32); qs = np.empty(x.size, np.int8); bs = np.empty(nb * 16, np.int16)
    lib().pmo_quantize_q8k(_p(x), x.size, _p(d), _p(qs), _p(bs))
    return d, qs, bs


def quantize_q8_0_act(x: np.ndarray):
    x = _c(x, np.float32).ravel()
    nb = x.size // 32
    d = np.empty(nb, np.uint16); qs = np.empty(x.size, np.int8)
    lib().pmo_quantize_q8_0_act(_p(x), x.size, _p(d), _p(qs))
    return d.view(np.float16), qs


def qmatmul(dtype: int, w_blocks: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1, cols)
    w_blocks = _c(w_blocks, np.uint8)
    y = np.empty((x.shape[0], rows), np.float32)
    if lib().pmo_qmatmul(dtype, _p(w_blocks), rows, cols, _p(x), x.shape[0], _p(y)):
        raise ValueError("pmo_qmatmul failed")
    return y


def rms_norm(x: np.ndarray, weight, eps: float) -> np.ndarray:
    x = _c(x, np.float32)
    n, H = x.shape
    w = None if weight is None else _c(weight, np.float32)
    y = np.empty_like(x)
    lib().pmo_rms_norm(_p(x), _p(w), n, H, eps, _p(y))
    return y


class Layer:
    """Host copy of one MoE block's tensors (numpy arrays of raw GGUF block bytes)."""

    def __init__(self, H, F, E, k, gate, up, down, gate_dtype, up_dtype, down_dtype, router_w,
                 shared=None, router_bias=None, router_dtype=0, router_q=None):
        self.H, self.F, self.E, self.k = H, F, E, k
        self.gate, self.up, self.down = (_c(a, np.uint8) for a in (gate, up, down))
        self.gate_dtype, self.up_dtype, self.down_dtype = gate_dtype, up_dtype, down_dtype
        self.router_w = _c(router_w, np.float32)
        self.router_bias = None if router_bias is None else _c(router_bias, np.float32)
        self.shared = None
        if shared is not None:
            self.shared = dict(shared)
            for key in ("gate", "up", "down"):
                self.shared[key] = _c(self.shared[key], np.uint8)
            self.shared["gate_inp"] = _c(self.shared["gate_inp"], np.float32)
        s = _Layer()
        s.H, s.F, s.E, s.k = H, F, E, k
        s.gate_dtype, s.up_dtype, s.down_dtype = gate_dtype, up_dtype, down_dtype
        s.gate_exps, s.up_exps, s.down_exps = (a.ctypes.data for a in (self.gate, self.up, self.down))
        s.has_shared = 0 if self.shared is None else 1
        if self.shared is not None:
            s.sh_gate_dtype, s.sh_up_dtype, s.sh_down_dtype = (
                self.shared["gate_dtype"], self.shared["up_dtype"], self.shared["down_dtype"])
            s.sh_gate, s.sh_up, s.sh_down = (self.shared[key].ctypes.data for key in ("gate", "up", "down"))
            s.sh_gate_inp = self.shared["gate_inp"].ctypes.data
        s.router_w = self.router_w.ctypes.data
        s.router_bias = None if self.router_bias is None else self.router_bias.ctypes.data
        # a quantised router: raw blocks [E, H / block] of type router_dtype (router_w stays as the f32 it was made from)
        self.router_dtype = int(router_dtype)
        self.router_q = None if router_q is None else _c(router_q, np.uint8)
        s.router_dtype = self.router_dtype if self.router_q is not None else 0
        s.router_q = None if self.router_q is None else self.router_q.ctypes.data
        self._s = s

    # -- pieces -----------------------------------------------------------------
    def router_logits(self, x):
        x = _c(x, np.float32).reshape(-1, self.H)
        out = np.empty((x.shape[0], self.E), np.float32)
        rc = lib().pmo_layer_router_logits(C.byref(self._s), _p(x), x.shape[0], _p(out))
        if rc:
            raise RuntimeError(f"pmo_layer_router_logits failed ({rc})")
        return out

    def route_topk(self, logits, with_probs=False):
        logits = _c(logits, np.float32).reshape(-1, self.E)
        n = logits.shape[0]
        idx = np.empty((n, self.k), np.uint32); w = np.empty((n, self.k), np.float32)
        probs = np.empty((n, self.E), np.float32) if with_probs else None
        lib().pmo_route_topk(_p(logits), n, self.E, self.k, _p(idx), _p(w), _p(probs))
        return (idx, w, probs) if with_probs else (idx, w)

    def router_stats(self, logits, idx):
        """(expert_counts [E], z, lb) of one block: the per-block terms of compute_z_loss and
        compute_load_balance_loss (paramecia-model/src/qwen3_next.rs:5549-5648), in float64."""
        logits = np.asarray(logits, np.float64).reshape(-1, self.E)
        idx = np.asarray(idx).reshape(logits.shape[0], -1).astype(np.int64)
        mx = logits.max(-1, keepdims=True)
        ex = np.exp(logits - mx)
        lse = mx[:, 0] + np.log(ex.sum(-1))
        z = float(np.mean(lse * lse))                                   # mean(log_sum_exp^2), 5573
        probs = ex / ex.sum(-1, keepdims=True)                           # softmax_last_dim, 5617
        sel = idx[(idx >= 0) & (idx < self.E)]                           # ids past E are skipped, 5624
        counts = np.bincount(sel, minlength=self.E).astype(np.float64)
        f = counts / idx.size                                            # / total_selections, 5629-5634
        lb = float(self.E * np.sum(f * probs.mean(0)))                   # E * sum(f_i * p_i), 5641-5645
        return counts, z, lb

    def experts_forward(self, x, idx, w):
        x = _c(x, np.float32).reshape(-1, self.H)
        idx = _c(idx, np.uint32); w = _c(w, np.float32)
        out = np.empty_like(x)
        if lib().pmo_experts_forward(C.byref(self._s), _p(x), x.shape[0], _p(idx), _p(w), idx.shape[1], _p(out)):
            raise ValueError("pmo_experts_forward failed")
        return out

    def shared_forward(self, x):
        x = _c(x, np.float32).reshape(-1, self.H)
        out = np.empty_like(x)
        if lib().pmo_shared_forward(C.byref(self._s), _p(x), x.shape[0], _p(out)):
            raise ValueError("pmo_shared_forward failed")
        return out

    # -- whole block ------------------------------------------------------------
    def forward(self, x):
        """MoeBlock::forward_with_stats: returns (out, logits (unclamped), top_idx, top_w)."""
        x = _c(x, np.float32).reshape(-1, self.H)
        n = x.shape[0]
        out = np.empty_like(x)
        logits = np.empty((n, self.E), np.float32)
        idx = np.empty((n, self.k), np.uint32); w = np.empty((n, self.k), np.float32)
        if lib().pmo_moe_forward(C.byref(self._s), _p(x), n, _p(out), _p(logits), _p(idx), _p(w)):
            raise ValueError("pmo_moe_forward failed")
        return out, logits, idx, w

    def forward_exact(self, x, idx, w):
        x = _c(x, np.float32).reshape(-1, self.H)
        idx = _c(idx, np.uint32); w = _c(w, np.float32)
        out = np.empty_like(x)
        lib().pmo_moe_forward_exact(C.byref(self._s), _p(x), x.shape[0], _p(idx), _p(w), _p(out))
        return out
