"""Shared helpers of the test-suite: the oracle side of a synthetic layer and error metrics."""
import numpy as np
import torch

from oracle import pmoe_oracle as po


def oracle_layer(t) -> "po.Layer":
    """The CPU oracle's view of a paramecia_b200.synth.make_layer() dict (same bytes)."""
    def u8(x):
        return x.detach().cpu().numpy()
    shared = None
    if t["shared"] is not None:
        s = t["shared"]
        shared = dict(gate=u8(s["gate"]), up=u8(s["up"]), down=u8(s["down"]), gate_dtype=s["gate_dtype"],
                      up_dtype=s["up_dtype"], down_dtype=s["down_dtype"], gate_inp=s["gate_inp"].cpu().numpy())
    bias = None if t["router_bias"] is None else t["router_bias"].cpu().numpy()
    return po.Layer(t["H"], t["F"], t["E"], t["k"], u8(t["gate"]), u8(t["up"]), u8(t["down"]),
                    t["gate_dtype"], t["up_dtype"], t["down_dtype"], t["router_w"].cpu().numpy(),
                    shared=shared, router_bias=bias, router_dtype=t.get("router_dtype") or 0,
                    router_q=None if t.get("router_q") is None else u8(t["router_q"]))


def rel_l2(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def max_abs(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


# required tolerance for layer outputs in fp32 accumulation
MAX_ABS_TOL = 2e-2
REL_L2_TOL = 1e-3


def seeded_x(n, H, seed, dtype=torch.float32):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn((n, H), generator=g, dtype=torch.float32)
    return x.to(dtype)
