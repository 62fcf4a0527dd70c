"""Seeded synthetic MoE layers in GGUF block formats.

The reference publishes no benchmark data for this path, so the workloads are synthetic:
normal weights N(0, 0.02) quantised to Q2_K ... Q6_K / Q8_0 blocks, a float router and normal
inputs.  The quantisers here are plain torch tensor code (CPU or CUDA) used only to
manufacture valid blocks; the library and the CPU oracle both consume the resulting bytes,
so their quality does not enter any comparison.  Q8_0 follows the ggml reference quantiser;
the K-quants are simple min/max quantisers.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ._lib import Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_0

PRESETS = {
    # name: (gate/up dtype, down dtype, shared dtype)
    "q4k": (Q4_K, Q4_K, Q4_K),          # every matrix Q4_K
    "q4k_m": (Q4_K, Q6_K, Q8_0),        # Q4_K_M-style mix: gate/up Q4_K, down Q6_K, shared Q8_0
    "q4k_q6k": (Q4_K, Q6_K, Q6_K),
    "q4k_q6k_all": (Q4_K, Q6_K, (Q4_K, Q6_K)),  # shared expert quantised like the routed ones
    "q8_0": (Q8_0, Q8_0, Q8_0),
    "q6k": (Q6_K, Q6_K, Q6_K),
    "q5k": (Q5_K, Q5_K, Q5_K),
    "q5k_m": (Q5_K, Q6_K, Q8_0),        # Q5_K_M-style mix
    "q2k": (Q2_K, Q2_K, Q2_K),
    "q3k": (Q3_K, Q3_K, Q3_K),
    "q3k_m": (Q3_K, Q4_K, Q8_0),        # Q3_K_M-style mix
    "q2k_q3k": (Q2_K, Q3_K, Q4_K),
}


def _half_bytes(v: torch.Tensor) -> torch.Tensor:
    return v.to(torch.float16).contiguous().view(torch.uint8).reshape(v.shape[0], 2)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 32).float()
    amax = xb.abs().amax(-1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(xb * inv[:, None]).clamp(-127, 127).to(torch.int8)
    return torch.cat([_half_bytes(d), q.view(torch.uint8)], dim=1).reshape(-1)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 8, 32).float()
    nb = xb.shape[0]
    mn = xb.amin(-1).clamp(max=0)
    mx = xb.amax(-1).clamp(min=0)
    scales = (mx - mn) / 15.0
    mins = -mn
    max_scale = scales.amax(-1)
    max_min = mins.amax(-1)
    inv_s = torch.where(max_scale > 0, 63.0 / max_scale, torch.zeros_like(max_scale))
    inv_m = torch.where(max_min > 0, 63.0 / max_min, torch.zeros_like(max_min))
    ls = torch.round(inv_s[:, None] * scales).clamp(0, 63).to(torch.int32)
    lm = torch.round(inv_m[:, None] * mins).clamp(0, 63).to(torch.int32)
    d16 = (max_scale / 63.0).to(torch.float16)
    m16 = (max_min / 63.0).to(torch.float16)
    dq = d16.float()[:, None] * ls.float()
    mq = m16.float()[:, None] * lm.float()
    q = torch.where(dq[..., None] > 0, torch.round((xb + mq[..., None]) / dq[..., None].clamp(min=1e-30)),
                    torch.zeros_like(xb)).clamp(0, 15).to(torch.uint8)
    q = q.reshape(nb, 4, 2, 32)
    qs = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(nb, 128)
    sb = torch.empty((nb, 12), dtype=torch.int32, device=x.device)
    sb[:, 0:4] = ls[:, 0:4] | ((ls[:, 4:8] >> 4) << 6)
    sb[:, 4:8] = lm[:, 0:4] | ((lm[:, 4:8] >> 4) << 6)
    sb[:, 8:12] = (ls[:, 4:8] & 0xF) | ((lm[:, 4:8] & 0xF) << 4)
    return torch.cat([_half_bytes(d16), _half_bytes(m16), sb.to(torch.uint8), qs], dim=1).reshape(-1)


def _pack_2bit(q: torch.Tensor) -> torch.Tensor:
    """[nb, 256] values 0..3 -> [nb, 64] bytes: element 128*half + 32*stream + l in byte 32*half + l at bits 2*stream."""
    q = q.reshape(-1, 2, 4, 32).to(torch.uint8)
    out = q[:, :, 0] | (q[:, :, 1] << 2) | (q[:, :, 2] << 4) | (q[:, :, 3] << 6)
    return out.reshape(-1, 64)


def quantize_q2_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 16, 16).float()
    mn = xb.amin(-1).clamp(max=0)
    mx = xb.amax(-1).clamp(min=0)
    scales = (mx - mn) / 3.0
    mins = -mn
    max_scale = scales.amax(-1)
    max_min = mins.amax(-1)
    inv_s = torch.where(max_scale > 0, 15.0 / max_scale, torch.zeros_like(max_scale))
    inv_m = torch.where(max_min > 0, 15.0 / max_min, torch.zeros_like(max_min))
    ls = torch.round(inv_s[:, None] * scales).clamp(0, 15).to(torch.int32)
    lm = torch.round(inv_m[:, None] * mins).clamp(0, 15).to(torch.int32)
    d16 = (max_scale / 15.0).to(torch.float16)
    m16 = (max_min / 15.0).to(torch.float16)
    dq = d16.float()[:, None] * ls.float()
    mq = m16.float()[:, None] * lm.float()
    q = torch.where(dq[..., None] > 0, torch.round((xb + mq[..., None]) / dq[..., None].clamp(min=1e-30)),
                    torch.zeros_like(xb)).clamp(0, 3)
    sc = (ls | (lm << 4)).to(torch.uint8)
    return torch.cat([sc, _pack_2bit(q.reshape(-1, 256)), _half_bytes(d16), _half_bytes(m16)], dim=1).reshape(-1)


def quantize_q3_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 16, 16).float()
    nb = xb.shape[0]
    scales = xb.abs().amax(-1) / 4.0
    max_scale = scales.amax(-1)
    inv = torch.where(max_scale > 0, 31.0 / max_scale, torch.zeros_like(max_scale))
    d16 = (max_scale / 31.0).to(torch.float16)
    s = torch.round(inv[:, None] * scales).clamp(0, 31).to(torch.int32)
    dq = d16.float()[:, None] * s.float()
    q = torch.where(dq[..., None] > 0, torch.round(xb / dq[..., None].clamp(min=1e-30)), torch.zeros_like(xb)).clamp(-4, 3)
    u = (q + 4).to(torch.uint8).reshape(nb, 256)            # 0..7: low two bits in qs, the third in hmask
    hb = (u >> 2).reshape(nb, 2, 4, 32)                      # [block, half, stream, l]
    hmask = torch.zeros((nb, 32), dtype=torch.uint8, device=x.device)
    for h in range(2):
        for g in range(4):
            hmask |= hb[:, h, g] << (4 * h + g)
    l6 = s + 32                                              # stored with an offset of 32
    sb = torch.zeros((nb, 12), dtype=torch.int32, device=x.device)
    sb[:, 0:8] = (l6[:, 0:8] & 0xF) | ((l6[:, 8:16] & 0xF) << 4)
    for j in range(16):
        sb[:, 8 + j % 4] |= (l6[:, j] >> 4) << (2 * (j // 4))
    return torch.cat([hmask, _pack_2bit(u & 3), sb.to(torch.uint8), _half_bytes(d16)], dim=1).reshape(-1)


def quantize_q5_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 8, 32).float()
    nb = xb.shape[0]
    mn = xb.amin(-1).clamp(max=0)
    mx = xb.amax(-1).clamp(min=0)
    scales = (mx - mn) / 31.0
    mins = -mn
    max_scale = scales.amax(-1)
    max_min = mins.amax(-1)
    inv_s = torch.where(max_scale > 0, 63.0 / max_scale, torch.zeros_like(max_scale))
    inv_m = torch.where(max_min > 0, 63.0 / max_min, torch.zeros_like(max_min))
    ls = torch.round(inv_s[:, None] * scales).clamp(0, 63).to(torch.int32)
    lm = torch.round(inv_m[:, None] * mins).clamp(0, 63).to(torch.int32)
    d16 = (max_scale / 63.0).to(torch.float16)
    m16 = (max_min / 63.0).to(torch.float16)
    dq = d16.float()[:, None] * ls.float()
    mq = m16.float()[:, None] * lm.float()
    q = torch.where(dq[..., None] > 0, torch.round((xb + mq[..., None]) / dq[..., None].clamp(min=1e-30)),
                    torch.zeros_like(xb)).clamp(0, 31).to(torch.uint8)
    q = q.reshape(nb, 4, 2, 32)   # [block, 64-group, low/high sub-block, l]
    qs = ((q[:, :, 0, :] & 0xF) | ((q[:, :, 1, :] & 0xF) << 4)).reshape(nb, 128)
    qh = torch.zeros((nb, 32), dtype=torch.uint8, device=x.device)
    for g in range(4):   # bit 2g: low sub-block of group g, bit 2g+1: its high sub-block
        qh |= (q[:, g, 0, :] >> 4) << (2 * g)
        qh |= (q[:, g, 1, :] >> 4) << (2 * g + 1)
    sb = torch.empty((nb, 12), dtype=torch.int32, device=x.device)
    sb[:, 0:4] = ls[:, 0:4] | ((ls[:, 4:8] >> 4) << 6)
    sb[:, 4:8] = lm[:, 0:4] | ((lm[:, 4:8] >> 4) << 6)
    sb[:, 8:12] = (ls[:, 4:8] & 0xF) | ((lm[:, 4:8] & 0xF) << 4)
    return torch.cat([_half_bytes(d16), _half_bytes(m16), sb.to(torch.uint8), qh, qs], dim=1).reshape(-1)


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.reshape(-1, 16, 16).float()
    nb = xb.shape[0]
    scales = xb.abs().amax(-1) / 31.0
    max_scale = scales.amax(-1)
    inv = torch.where(max_scale > 0, 127.0 / max_scale, torch.zeros_like(max_scale))
    d16 = (max_scale / 127.0).to(torch.float16)
    s = torch.round(inv[:, None] * scales).clamp(0, 127)
    dq = d16.float()[:, None] * s
    q = torch.where(dq[..., None] > 0, torch.round(xb / dq[..., None].clamp(min=1e-30)), torch.zeros_like(xb))
    L = (q.clamp(-32, 31) + 32).to(torch.uint8).reshape(nb, 2, 4, 32)
    q1, q2, q3, q4 = L[:, :, 0], L[:, :, 1], L[:, :, 2], L[:, :, 3]
    ql = torch.stack([(q1 & 0xF) | ((q3 & 0xF) << 4), (q2 & 0xF) | ((q4 & 0xF) << 4)], dim=2).reshape(nb, 128)
    qh = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).reshape(nb, 64)
    return torch.cat([ql, qh, s.to(torch.int8).view(torch.uint8), _half_bytes(d16)], dim=1).reshape(-1)


_QUANT = {Q8_0: quantize_q8_0, Q2_K: quantize_q2_k, Q3_K: quantize_q3_k, Q4_K: quantize_q4_k, Q5_K: quantize_q5_k,
          Q6_K: quantize_q6_k}


def quantize(x: torch.Tensor, dtype: int, chunk_elems: int = 1 << 26) -> torch.Tensor:
    """f32 tensor (element count a multiple of the block size) -> raw GGUF blocks (uint8)."""
    flat = x.reshape(-1)
    parts = [_QUANT[dtype](flat[i:i + chunk_elems]) for i in range(0, flat.numel(), chunk_elems)]
    return parts[0] if len(parts) == 1 else torch.cat(parts)


def random_quantized(shape, dtype: int, gen: torch.Generator, device, std: float = 0.02,
                     chunk_rows: int = 64) -> torch.Tensor:
    """N(0, std) weights of `shape` quantised to `dtype`, generated chunk by chunk along dim 0."""
    rows = shape[0]
    inner = 1
    for s in shape[1:]:
        inner *= s
    parts = []
    for r0 in range(0, rows, chunk_rows):
        r = min(chunk_rows, rows - r0)
        w = torch.randn((r, inner), generator=gen, device=device, dtype=torch.float32) * std
        parts.append(quantize(w, dtype))
    return torch.cat(parts)


def zipf_router_bias(E: int, seed: int, device="cpu") -> torch.Tensor:
    """b_e = 2 * ln(1 / rank_e) with rank a seeded permutation of 1..E (skewed expert load)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    rank = torch.randperm(E, generator=g) + 1
    return (2.0 * torch.log(1.0 / rank.float())).to(device)


def make_layer(H=2048, F=512, E=512, k=10, preset="q4k_m", seed=0, device="cpu", shared=True,
               zipf=False, layer=0, router_dtype: Optional[int] = None) -> Dict[str, object]:
    """One synthetic MoE block as raw tensors.  Returns a dict with the GGUF block bytes
    (uint8 tensors on `device`), dtypes and the float tensors.  `router_dtype` (a block type) also gives the
    router quantised: `router_q`, blocks [E, H / block] made from `router_w`."""
    gu_dt, dn_dt, sh_dt = PRESETS[preset]
    sh_gu, sh_dn = sh_dt if isinstance(sh_dt, tuple) else (sh_dt, sh_dt)
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0x5EED0000 + 1000 * layer + seed)
    t = dict(H=H, F=F, E=E, k=k, preset=preset,
             gate_dtype=gu_dt, up_dtype=gu_dt, down_dtype=dn_dt,
             gate=random_quantized((E, F * H), gu_dt, gen, dev),
             up=random_quantized((E, F * H), gu_dt, gen, dev),
             down=random_quantized((E, H * F), dn_dt, gen, dev),
             router_w=torch.randn((E, H), generator=gen, device=dev) * 0.02,
             router_bias=zipf_router_bias(E, seed + 17, dev) if zipf else None,
             shared=None)
    t["router_dtype"] = router_dtype
    t["router_q"] = None if router_dtype is None else quantize(t["router_w"].float(), router_dtype)
    if shared:
        t["shared"] = dict(gate_dtype=sh_gu, up_dtype=sh_gu, down_dtype=sh_dn,
                           gate=random_quantized((1, F * H), sh_gu, gen, dev),
                           up=random_quantized((1, F * H), sh_gu, gen, dev),
                           down=random_quantized((1, H * F), sh_dn, gen, dev),
                           gate_inp=torch.randn((H,), generator=gen, device=dev) * 0.02)
    return t


def make_block(t: Dict[str, object], device="cuda:0", max_tokens=256, expert_base=0, E_local: Optional[int] = None,
               training_mode=False, ep_rank=0, ep_size=0):
    """Builds a MoeBlock from make_layer() output; an expert slice gives one expert-parallel rank."""
    from .moe import MoeBlock, QTensor, SharedExpertWeights
    H, F, E, k = t["H"], t["F"], t["E"], t["k"]
    El = E if E_local is None else E_local

    def sl(name, dtype, rows, cols):
        from ._lib import row_bytes
        per = rows * row_bytes(dtype, cols)
        return QTensor(t[name][expert_base * per:(expert_base + El) * per], dtype, (El, rows, cols))

    sh = None
    if t["shared"] is not None:
        s = t["shared"]
        sh = SharedExpertWeights(QTensor(s["gate"], s["gate_dtype"], (F, H)), QTensor(s["up"], s["up_dtype"], (F, H)),
                                 QTensor(s["down"], s["down_dtype"], (H, F)), s["gate_inp"])
    router = t["router_w"] if t.get("router_q") is None else QTensor(t["router_q"], t["router_dtype"], (E, H))
    return MoeBlock(sl("gate", t["gate_dtype"], F, H), sl("up", t["up_dtype"], F, H), sl("down", t["down_dtype"], H, F),
                    router, k, shared_expert=sh, device=device, max_tokens=max_tokens,
                    router_bias=t["router_bias"], num_experts=E, expert_base=expert_base,
                    training_mode=training_mode, ep_rank=ep_rank, ep_size=ep_size)


def make_rank_block(t: Dict[str, object], device, max_tokens: int, rank: int, world: int, placement: str = "contiguous"):
    """The MoeBlock of rank `rank` of `world` expert-parallel ranks: E / world routed experts, contiguous
    (rank * E/world ...) or round-robin (rank, rank + world, ...), router and shared expert whole."""
    from .moe import MoeBlock, QTensor, SharedExpertWeights
    from ._lib import row_bytes
    H, F, E, k = t["H"], t["F"], t["E"], t["k"]
    if world <= 1:
        return make_block(t, device, max_tokens=max_tokens)
    El = E // world
    if placement == "contiguous":
        return make_block(t, device, max_tokens=max_tokens, expert_base=rank * El, E_local=El, ep_rank=rank, ep_size=world)

    def pick(name, dtype, rows, cols):   # experts rank, rank + world, ... gathered into one tensor
        per = rows * row_bytes(dtype, cols)
        return QTensor(t[name].reshape(E, per)[rank::world].contiguous().reshape(-1), dtype, (El, rows, cols))

    sh = None
    if t["shared"] is not None:
        s = t["shared"]
        sh = SharedExpertWeights(QTensor(s["gate"], s["gate_dtype"], (F, H)), QTensor(s["up"], s["up_dtype"], (F, H)),
                                 QTensor(s["down"], s["down_dtype"], (H, F)), s["gate_inp"])
    return MoeBlock(pick("gate", t["gate_dtype"], F, H), pick("up", t["up_dtype"], F, H), pick("down", t["down_dtype"], H, F),
                    t["router_w"], k, shared_expert=sh, device=device, max_tokens=max_tokens,
                    router_bias=t["router_bias"], num_experts=E, ep_rank=rank, ep_size=world, ep_placement="round_robin")


def layer_bytes(t: Dict[str, object]) -> int:
    n = sum(t[k].numel() for k in ("gate", "up", "down")) + t["router_w"].numel() * 4
    if t["shared"] is not None:
        n += sum(t["shared"][k].numel() for k in ("gate", "up", "down"))
    return n


def expected_distinct(E: int, k: int, n: int) -> float:
    """Expected number of distinct experts hit by n tokens under uniform routing."""
    return E * (1.0 - math.pow(1.0 - k / E, n))
