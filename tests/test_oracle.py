"""CPU tests of the oracle: block codecs against the gguf-py golden vectors, the activation
quantisers and block dots against straight numpy restatements, routing tie rules, and the
whole-block oracle against its exact-arithmetic variant."""
import os

import numpy as np
import pytest
import torch

from oracle import pmoe_oracle as po
from paramecia_b200 import synth
from tests.common import oracle_layer, rel_l2, seeded_x

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "codec_golden.npz"))
LG = np.load(os.path.join(os.path.dirname(__file__), "golden", "layer_golden.npz"))
DT = {"q2_k": po.Q2_K, "q3_k": po.Q3_K, "q4_k": po.Q4_K, "q5_k": po.Q5_K, "q6_k": po.Q6_K, "q8_0": po.Q8_0}


@pytest.mark.parametrize("name", ["q2_k", "q3_k", "q4_k", "q5_k", "q6_k", "q8_0"])
def test_dequantize_matches_gguf_py_bit_exact(name):
    raw, want = G[name + "_blocks"], G[name + "_dequant"]
    got = po.dequantize(DT[name], raw.reshape(-1), want.size)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q8_0_quantiser_matches_gguf_py():
    got = po.quantize(po.Q8_0, G["q8_0_quant_in"])
    assert np.array_equal(got, G["q8_0_quant_blocks"])


@pytest.mark.parametrize("dtype,tol", [(po.Q2_K, 0.4), (po.Q3_K, 0.25), (po.Q4_K, 0.12), (po.Q5_K, 0.06), (po.Q6_K, 0.03),
                                       (po.Q8_0, 0.01)])
def test_weight_quantisers_round_trip(dtype, tol):
    rng = np.random.default_rng(1)
    w = (rng.standard_normal(256 * 32) * 0.02).astype(np.float32)
    for q in (po.quantize(dtype, w), synth.quantize(torch.from_numpy(w), dtype).numpy()):
        back = po.dequantize(dtype, q, w.size)
        assert rel_l2(back, w) < tol
    z = po.dequantize(dtype, po.quantize(dtype, np.zeros(256, np.float32)), 256)
    assert not z.any()


def test_q8k_activation_quantiser():
    rng = np.random.default_rng(2)
    x = rng.standard_normal(512).astype(np.float32)
    x[256:] = 0.0                      # an all-zero block gives d = 0
    x[5] = -7.0                        # the largest magnitude keeps its sign: iscale = -128 / max
    x[9] = 7.0                         # same magnitude later in the block must not win
    d, qs, bs = po.quantize_q8k(x)
    assert d[1] == 0 and not qs[256:].any() and not bs[16:].any()
    iscale = np.float32(-128.0) / np.float32(-7.0)
    want = np.minimum(np.sign(iscale * x[:256]) * np.floor(np.abs(iscale * x[:256]) + 0.5), 127).astype(np.int8)
    assert np.array_equal(qs[:256], want)
    assert qs[5] == -128 and qs[9] == 127
    assert d[0] == np.float32(1.0) / iscale
    assert np.array_equal(bs[:16], want.reshape(16, 16).astype(np.int32).sum(1).astype(np.int16))


def test_q8_0_activation_quantiser():
    rng = np.random.default_rng(3)
    x = rng.standard_normal(64).astype(np.float32)
    x[32:] = 0
    d, qs = po.quantize_q8_0_act(x)
    amax = np.abs(x[:32]).max()
    dd = np.float32(amax) / np.float32(127)
    assert d[0] == np.float16(dd) and d[1] == 0
    q = x[:32] * (np.float32(1) / dd)
    assert np.array_equal(qs[:32], (np.sign(q) * np.floor(np.abs(q) + 0.5)).astype(np.int8))


@pytest.mark.parametrize("dtype", [po.Q2_K, po.Q3_K, po.Q4_K, po.Q5_K, po.Q6_K, po.Q8_0])
def test_qmatmul_is_integer_dot_of_quantised_activations(dtype):
    rng = np.random.default_rng(4)
    rows, cols, m = 8, 512, 3
    w = po.quantize(dtype, (rng.standard_normal(rows * cols) * 0.02).astype(np.float32))
    x = rng.standard_normal((m, cols)).astype(np.float32)
    got = po.qmatmul(dtype, w, rows, cols, x)
    wd = po.dequantize(dtype, w, rows * cols).reshape(rows, cols).astype(np.float64)
    xq = np.empty_like(x, dtype=np.float64)   # the activations as the reference CPU path sees them
    for r in range(m):
        if dtype == po.Q8_0:
            d, qs = po.quantize_q8_0_act(x[r])
            xq[r] = qs.reshape(-1, 32) .astype(np.float64).reshape(-1) * np.repeat(d.astype(np.float64), 32)
        else:
            d, qs, _ = po.quantize_q8k(x[r])
            xq[r] = qs.astype(np.float64) * np.repeat(d.astype(np.float64), 256)
    want = xq @ wd.T
    assert rel_l2(got, want) < 2e-6
    assert rel_l2(got, x.astype(np.float64) @ wd.T) > 1e-3   # and NOT the unquantised product


def test_router_order_and_topk_ties():
    E, H, k = 16, 256, 4
    rng = np.random.default_rng(5)
    W = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    W[7] = W[2]; W[11] = W[2]
    L = po.Layer(H, 256, E, k, np.zeros(E * 256 * 144 // 256 * H // 1, np.uint8)[:E * 256 * (H // 256) * 144],
                 np.zeros(E * 256 * (H // 256) * 144, np.uint8), np.zeros(E * H * 144, np.uint8),
                 po.Q4_K, po.Q4_K, po.Q4_K, W)
    x = rng.standard_normal((5, H)).astype(np.float32)
    x[0] = W[2] * 500        # makes experts 2, 7, 11 the (tied) winners of token 0
    logits = L.router_logits(x)
    np.testing.assert_allclose(logits, x @ W.T, rtol=0, atol=2e-5)
    assert np.array_equal(logits[:, 2], logits[:, 7]) and np.array_equal(logits[:, 2], logits[:, 11])
    idx, w, probs = L.route_topk(logits, with_probs=True)
    assert list(idx[0][:3]) == [2, 7, 11]            # equal probabilities keep ascending expert order
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)
    assert (np.diff(w, axis=1) <= 0).all()          # descending weights
    huge = np.full((1, E), 1000.0, np.float32); huge[0, 3] = -1000.0
    i2, w2 = L.route_topk(huge)                     # clamp to +-100 keeps softmax finite
    assert np.isfinite(w2).all() and 3 not in i2[0]


@pytest.mark.parametrize("preset", ["q4k", "q4k_m", "q8_0"])
def test_block_oracle_vs_exact_and_golden(preset):
    t = synth.make_layer(E=8, k=2, preset=preset, seed=5)
    ol = oracle_layer(t)
    x = seeded_x(3, 2048, 9).numpy()
    out, logits, idx, w = ol.forward(x)
    assert np.array_equal(idx, LG[preset + "_idx"])
    np.testing.assert_allclose(out, LG[preset + "_out"], rtol=0, atol=2e-6)
    exact = ol.forward_exact(x, idx, w)
    r = rel_l2(out, exact)
    assert 1e-3 < r < 5e-2    # activation quantisation is visible but small
    # pieces add up: routed + shared
    parts = ol.experts_forward(x, idx, w) + ol.shared_forward(x)
    np.testing.assert_allclose(parts, out, rtol=0, atol=1e-6)


def test_rms_norm():
    x = seeded_x(4, 2048, 3).numpy()
    wt = np.linspace(0.5, 1.5, 2048).astype(np.float32)
    y = po.rms_norm(x, wt, 1e-6)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6) * wt
    np.testing.assert_allclose(y, want, rtol=2e-6)


def test_router_stats_formulas():
    # the oracle's statistics against the formulas written with torch ops, as the reference writes them
    import torch
    from paramecia_b200 import synth
    from tests.common import oracle_layer
    t = synth.make_layer(E=16, k=3, preset="q8_0", seed=2, shared=False)
    ol = oracle_layer(t)
    rng = np.random.default_rng(4)
    logits = rng.standard_normal((25, 16)).astype(np.float32) * 3
    idx = np.stack([rng.choice(16, size=3, replace=False) for _ in range(25)]).astype(np.uint32)
    counts, z, lb = ol.router_stats(logits, idx)
    L = torch.from_numpy(logits).double()
    lse = torch.logsumexp(L, -1)
    assert abs(z - float((lse * lse).mean())) < 1e-12
    f = torch.bincount(torch.from_numpy(idx.astype(np.int64)).flatten(), minlength=16).double() / idx.size
    p = torch.softmax(L, -1).mean(0)
    assert abs(lb - float(16 * (f * p).sum())) < 1e-12
    assert counts.sum() == idx.size


@pytest.mark.parametrize("dtype", [po.Q2_K, po.Q3_K, po.Q4_K, po.Q5_K, po.Q6_K, po.Q8_0])
def test_modify_block_scales(dtype):
    """Block-scale multipliers (QTensor::modify_block_scales, qwen3_next.rs:1604-1606): the block's values times m,
    with the f16 scales re-rounded; quants untouched."""
    rng = np.random.default_rng(11)
    bs, ts, nb = po.block_size(dtype), po.type_size(dtype), 24
    w = po.quantize(dtype, (rng.standard_normal(nb * bs) * 0.02).astype(np.float32))
    ones = po.modify_block_scales(dtype, w, np.ones(nb, np.float32))
    assert np.array_equal(ones, w)                                        # m = 1 changes no byte
    m = np.array([2.0, 4.0, -1.0, 0.0] * (nb // 4), np.float32)           # exact in f16 (no subnormal is halved)
    got = po.dequantize(dtype, po.modify_block_scales(dtype, w, m), nb * bs)
    want = po.dequantize(dtype, w, nb * bs) * np.repeat(m, bs)
    assert np.array_equal(got, want)
    m = rng.uniform(0.5, 1.5, nb).astype(np.float32)                      # general: within f16 rounding of the scales
    mod = po.modify_block_scales(dtype, w, m)
    got = po.dequantize(dtype, mod, nb * bs)
    want = po.dequantize(dtype, w, nb * bs).astype(np.float64) * np.repeat(m.astype(np.float64), bs)
    assert np.max(np.abs(got - want)) <= 2.0 ** -10 * np.max(np.abs(want)) * 2
    # only the scale fields differ
    offs = {po.Q2_K: (80, 82), po.Q3_K: (108,), po.Q4_K: (0, 2), po.Q5_K: (0, 2), po.Q6_K: (208,), po.Q8_0: (0,)}[dtype]
    keep = np.ones(ts, bool)
    for o in offs:
        keep[o:o + 2] = False
    assert np.array_equal(mod.reshape(nb, ts)[:, keep], w.reshape(nb, ts)[:, keep])
    for o in offs:                                                         # and they are f16(f32(d) * m)
        d0 = w.reshape(nb, ts)[:, o:o + 2].copy().view(np.float16).astype(np.float32)[:, 0]
        d1 = mod.reshape(nb, ts)[:, o:o + 2].copy().view(np.float16)[:, 0]
        assert np.array_equal(d1, (d0 * m).astype(np.float16))


@pytest.mark.parametrize("dtype", [po.Q4_K, po.Q6_K, po.Q8_0])
def test_simd_block_dots_equal_the_portable_ones_bit_for_bit(dtype):
    rng = np.random.default_rng(17)
    rows, cols, m = 48, 2048, 5
    w = po.quantize(dtype, (rng.standard_normal(rows * cols) * 0.02).astype(np.float32))
    raw = w.reshape(-1, po.type_size(dtype)).copy()
    raw[3] = rng.integers(0, 256, raw.shape[1], dtype=np.uint8)     # arbitrary quants and sub-scales too
    off = {po.Q4_K: (0, 2), po.Q6_K: (208,), po.Q8_0: (0,)}[dtype]
    for o in off:
        raw[3, o:o + 2] = np.array([0.01], np.float16).view(np.uint8)
    w = raw.ravel()
    x = (rng.standard_normal((m, cols)) * 3).astype(np.float32)
    x[1, :300] = 0
    try:
        po.set_simd(True)
        a = po.qmatmul(dtype, w, rows, cols, x)
        assert "AVX2" in po.simd_kind()
        po.set_simd(False)
        b = po.qmatmul(dtype, w, rows, cols, x)
        assert "portable" in po.simd_kind()
    finally:
        po.set_simd(True)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_quantised_router_is_a_quantised_matmul():
    """A router held as GGUF blocks takes candle's quantised mat-mul (rows to Q8_K / Q8_0, integer block dots),
    not a dequantise-and-GEMV: the layer's logits are pmo_qmatmul of the router blocks, plus the bias."""
    rng = np.random.default_rng(5)
    E, H, F, k, n = 16, 256, 256, 3, 7
    wf = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    x = rng.standard_normal((n, H)).astype(np.float32)
    bias = rng.standard_normal(E).astype(np.float32)
    for dt in (po.Q8_0, po.Q4_K, po.Q6_K):
        rq = po.quantize(dt, wf)
        gate = po.quantize(po.Q4_K, (rng.standard_normal((E, F * H)) * 0.02).astype(np.float32))
        down = po.quantize(po.Q4_K, (rng.standard_normal((E, H * F)) * 0.02).astype(np.float32))
        L = po.Layer(H, F, E, k, gate, gate, down, po.Q4_K, po.Q4_K, po.Q4_K, wf, router_bias=bias,
                     router_dtype=dt, router_q=rq)
        want = po.qmatmul(dt, rq, E, H, x) + bias[None, :]
        got = L.router_logits(x)
        assert np.array_equal(got, want.astype(np.float32))
        # and it differs from the f32 router over the dequantised weights (the activations are quantised too)
        plain = po.Layer(H, F, E, k, gate, gate, down, po.Q4_K, po.Q4_K, po.Q4_K, po.dequantize(dt, rq, E * H).reshape(E, H),
                         router_bias=bias).router_logits(x)
        assert not np.array_equal(got, plain) and np.allclose(got, plain, atol=2e-2)
        out, logits, idx, w = L.forward(x)
        assert np.array_equal(logits, got)
