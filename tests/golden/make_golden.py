"""Generates tests/golden/codec_golden.npz.

The Rust reference cannot be built or run here (no cargo; its candle fork is not vendored) and
holds no golden vectors for this path, so the block codecs are pinned against an independent
implementation instead: the `gguf` Python package (gguf-py 0.19, the GGUF project's own
reader).  For seeded random Q2_K ... Q6_K / Q8_0 blocks (plus edge blocks: zero scales, largest
and negative f16 scales, all-ones payload) the file stores the raw block bytes and gguf-py's
dequantised f32 output, and for Q8_0 also gguf-py's quantisation of a seeded normal vector.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "codec_golden.npz")
SPECS = {"q4_k": (T.Q4_K, 144, (0, 2)), "q6_k": (T.Q6_K, 210, (208,)), "q8_0": (T.Q8_0, 34, (0,))}


def blocks(rng, nb, ts, scale_offsets):
    raw = rng.integers(0, 256, size=(nb, ts), dtype=np.uint8)
    for off in scale_offsets:
        v = raw[:, off:off + 2].copy().view(np.float16)
        v[~np.isfinite(v)] = np.float16(-0.75)
        v[0] = 0.0
        v[1] = np.float16(65504.0)
        v[2] = np.float16(-6.1e-5)
        raw[:, off:off + 2] = v.view(np.uint8)
    raw[3] = 0
    raw[4] = 255
    for off in scale_offsets:
        raw[4, off:off + 2] = np.array([1.0], np.float16).view(np.uint8)
    return raw


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    for name, (gt, ts, offs) in SPECS.items():
        raw = blocks(rng, 48, ts, offs)
        out[name + "_blocks"] = raw
        out[name + "_dequant"] = quants.dequantize(raw.reshape(-1), gt).astype(np.float32).reshape(-1)
    w = (rng.standard_normal(32 * 64) * 0.02).astype(np.float32)
    out["q8_0_quant_in"] = w
    out["q8_0_quant_blocks"] = quants.quantize(w, T.Q8_0).reshape(-1)
    # Q5_K joined later: its own generator, so that the entries above keep their values
    rng5 = np.random.default_rng(20240608)
    raw = blocks(rng5, 48, 176, (0, 2))
    out["q5_k_blocks"] = raw
    out["q5_k_dequant"] = quants.dequantize(raw.reshape(-1), T.Q5_K).astype(np.float32).reshape(-1)
    for seed, name, gt, ts, offs in ((20240609, "q2_k", T.Q2_K, 84, (80, 82)), (20240610, "q3_k", T.Q3_K, 110, (108,))):
        raw = blocks(np.random.default_rng(seed), 48, ts, offs)
        out[name + "_blocks"] = raw
        out[name + "_dequant"] = quants.dequantize(raw.reshape(-1), gt).astype(np.float32).reshape(-1)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()


def layer_goldens():
    """Outputs of the CPU oracle itself on small seeded layers (tests/golden/layer_golden.npz).
    They pin the oracle against accidental change; they are not reference outputs."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    from paramecia_b200 import synth
    from tests.common import oracle_layer, seeded_x
    out = {}
    for preset in ("q4k", "q4k_m", "q8_0"):
        t = synth.make_layer(E=8, k=2, preset=preset, seed=5)
        x = seeded_x(3, 2048, 9).numpy()
        y, logits, idx, w = oracle_layer(t).forward(x)
        out[preset + "_out"] = y
        out[preset + "_idx"] = idx
        out[preset + "_w"] = w
    path = os.path.join(os.path.dirname(OUT), "layer_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path)


if __name__ == "__main__":
    layer_goldens()
