"""GPU parity of the decode path against the CPU oracle, through the C ABI (ctypes binding).

Bars: router logits and top-k indices bit-exact; dequantised weights bit-exact; layer outputs
within max-abs 2e-2 and relative-L2 1e-3 of the oracle (the oracle quantises activations like
the reference CPU path, and so does the library, so the observed distance is far smaller).
"""
import os

import numpy as np
import pytest
import torch

from tests.common import MAX_ABS_TOL, REL_L2_TOL, max_abs, oracle_layer, rel_l2, seeded_x

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():  # collected on the CPU box too; every test here needs the GPU
    pytest.skip("needs a CUDA device", allow_module_level=True)

import paramecia_b200 as pm
from paramecia_b200 import synth
from oracle import pmoe_oracle as po

DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [pm.Q2_K, pm.Q3_K, pm.Q4_K, pm.Q5_K, pm.Q6_K, pm.Q8_0])
def test_dequantize_bit_exact(dtype):
    rng = np.random.default_rng(7)
    nb, ts, bs = 512, pm.type_size(dtype), pm.block_size(dtype)
    raw = rng.integers(0, 256, size=(nb, ts), dtype=np.uint8)
    offs = {pm.Q2_K: (80, 82), pm.Q3_K: (108,), pm.Q4_K: (0, 2), pm.Q5_K: (0, 2), pm.Q6_K: (208,), pm.Q8_0: (0,)}[dtype]
    for off in offs:  # keep the f16 scales finite; include zero, negative and large ones
        v = raw[:, off:off + 2].copy().view(np.float16)
        v[~np.isfinite(v)] = np.float16(-0.75)
        v[0] = 0.0
        v[1] = np.float16(65504.0)
        raw[:, off:off + 2] = v.view(np.uint8)
    raw[2] = 0
    raw[3, :] = 255
    if dtype in (pm.Q4_K, pm.Q5_K):
        raw[3, 0:4] = np.array([1.0, 1.0], np.float16).view(np.uint8)
    elif dtype == pm.Q2_K:
        raw[3, 80:84] = np.array([1.0, 1.0], np.float16).view(np.uint8)
    elif dtype == pm.Q3_K:
        raw[3, 108:110] = np.array([1.0], np.float16).view(np.uint8)
    elif dtype == pm.Q6_K:
        raw[3, 208:210] = np.array([1.0], np.float16).view(np.uint8)
    else:
        raw[3, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    want = po.dequantize(dtype, raw.ravel(), nb * bs)
    got = pm.dequantize(torch.from_numpy(raw.ravel()).to(DEV), dtype, nb * bs).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("n,xdtype", [(1, torch.float32), (7, torch.bfloat16), (64, torch.float32), (200, torch.bfloat16),
                                      (1000, torch.bfloat16), (530, torch.float32)])
def test_router_bit_exact(n, xdtype):
    t = synth.make_layer(E=512, k=10, preset="q8_0", seed=3, shared=False, H=2048, F=512)
    blk = synth.make_block(t, DEV, max_tokens=max(n, 256))
    x = seeded_x(n, 2048, 11, xdtype)
    logits, w, idx = blk.route(x.to(DEV))
    ol = oracle_layer(t)
    xf = x.float().numpy()
    want_logits = ol.router_logits(xf)
    want_idx, want_w = ol.route_topk(want_logits)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want_logits.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    np.testing.assert_allclose(w.cpu().numpy(), want_w, rtol=2e-6, atol=1e-9)
    blk.status()


@pytest.mark.parametrize("E", [64, 512])   # 512: the register-resident top-k kernel
def test_router_bias_and_ties(E):
    # identical router rows give exactly equal probabilities: the lower expert id must win
    t = synth.make_layer(E=E, k=4, preset="q8_0", seed=5, shared=False, F=512, zipf=True)
    t["router_w"][10] = t["router_w"][3]
    t["router_w"][40] = t["router_w"][3]
    t["router_bias"][10] = t["router_bias"][3]
    t["router_bias"][40] = t["router_bias"][3]
    blk = synth.make_block(t, DEV, max_tokens=64)
    x = seeded_x(33, 2048, 12)
    logits, w, idx = blk.route(x.to(DEV))
    ol = oracle_layer(t)
    want_logits = ol.router_logits(x.numpy())
    want_idx, want_w = ol.route_topk(want_logits)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want_logits.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)


CASES = [
    # preset, E, k, n, x dtype
    ("q4k", 512, 10, 1, torch.float32),       # benchmark configuration 1 (one f32 token, all Q4_K)
    ("q4k_m", 512, 10, 1, torch.bfloat16),    # benchmark configuration 2: the whole batch sweep 1 / 4 / 16 / 64
    ("q4k_m", 512, 10, 4, torch.bfloat16),
    ("q4k_m", 512, 10, 16, torch.bfloat16),
    ("q4k_m", 512, 10, 64, torch.bfloat16),
    ("q8_0", 64, 6, 17, torch.bfloat16),
    ("q6k", 16, 2, 3, torch.float32),
    ("q4k_q6k", 4, 1, 2, torch.float32),
    ("q4k_m", 32, 4, 130, torch.float32),     # many tokens per expert: several token passes
    ("q5k", 16, 3, 5, torch.float32),
    ("q5k_m", 64, 6, 40, torch.bfloat16),
    ("q2k", 16, 3, 5, torch.float32),
    ("q3k", 16, 3, 7, torch.float32),
    ("q3k_m", 64, 6, 40, torch.bfloat16),
    ("q2k_q3k", 32, 4, 70, torch.bfloat16),
]


@pytest.mark.parametrize("preset,E,k,n,xdtype", CASES)
def test_block_matches_oracle(preset, E, k, n, xdtype):
    t = synth.make_layer(E=E, k=k, preset=preset, seed=21, device=DEV if E >= 256 else "cpu")   # big layers are made on the GPU
    blk = synth.make_block(t, DEV, max_tokens=max(n, 8))
    x = seeded_x(n, 2048, 100 + n, xdtype)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    ol = oracle_layer(t)
    want, want_logits, want_idx, want_w = ol.forward(x.float().numpy())
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want_logits.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(got, want) <= REL_L2_TOL
    # The library repeats the oracle's integer arithmetic.  What remains is f32 re-association
    # and the rare activation whose int8 rounding flips because silu(gate)*up differs in its
    # last bit; that keeps the distance well inside the bar.
    assert rel_l2(got, want) <= 5e-4


@pytest.mark.parametrize("router_dtype,n,xdtype", [(8, 5, torch.float32), (12, 40, torch.bfloat16), (14, 700, torch.float32)])
def test_quantised_router(router_dtype, n, xdtype):
    """ffn_gate_inp held as Q8_0 / Q4_K / Q6_K blocks: the router is a quantised mat-mul like the experts'
    (models/with_tracing.rs:324-335).  The logits are integer block sums with f32 scales, so they match the oracle
    to f32 re-association; the seeded inputs have no near-ties, so the indices are equal."""
    t = synth.make_layer(E=64, k=6, preset="q4k_m", seed=31, router_dtype=router_dtype)
    blk = synth.make_block(t, DEV, max_tokens=max(n, 8))
    x = seeded_x(n, 2048, 300 + n, xdtype)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    ol = oracle_layer(t)
    want, want_logits, want_idx, _ = ol.forward(x.float().numpy())
    assert np.allclose(logits.cpu().numpy(), want_logits, rtol=1e-5, atol=1e-6)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL and rel_l2(got, want) <= 5e-4
    # the routing-only entry point takes the same path
    lg2, w2, idx2 = blk.route(x.to(DEV))
    assert torch.equal(lg2, logits.reshape(lg2.shape)) and torch.equal(idx2.reshape(idx.shape), idx)


def test_experts_and_shared_entry_points():
    t = synth.make_layer(E=32, k=4, preset="q4k_m", seed=8)
    blk = synth.make_block(t, DEV, max_tokens=32)
    ol = oracle_layer(t)
    x = seeded_x(9, 2048, 5)
    rng = np.random.default_rng(3)
    idx = np.stack([rng.choice(32, size=4, replace=False) for _ in range(9)]).astype(np.uint32)
    idx[0, 1] = 0xFFFFFFFF  # out-of-range ids are skipped (qwen3_next.rs:2045)
    idx[4, 0] = 32
    w = rng.random((9, 4)).astype(np.float32)
    got = blk.experts_forward_batched(x.to(DEV), torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w), 4)
    want = ol.experts_forward(x.numpy(), idx, w)
    assert rel_l2(got.cpu().numpy(), want) <= 5e-4
    got_s = blk.shared_forward(x.to(DEV)).cpu().numpy()
    want_s = ol.shared_forward(x.numpy())
    assert rel_l2(got_s, want_s) <= 5e-4
    # top_k smaller than the block's k
    got2 = blk.experts_forward_batched(x.to(DEV), torch.from_numpy(idx[:, :2].copy().view(np.int32)),
                                       torch.from_numpy(w[:, :2].copy()), 2)
    want2 = ol.experts_forward(x.numpy(), idx[:, :2].copy(), w[:, :2].copy())
    assert rel_l2(got2.cpu().numpy(), want2) <= 5e-4
    blk.status()


@pytest.mark.parametrize("n,begin,count,prefill,preset", [
    (23, 5, 11, "0", "q4k_q6k_all"), (23, 0, 23, "0", "q4k_q6k_all"), (23, 22, 1, "0", "q4k_q6k_all"),
    (150, 64, 70, "1", "q4k_q6k_all"), (9, 3, 0, "0", "q4k_q6k_all"),
    (150, 64, 70, "0", "q4k_m"),    # Q8_0 shared expert over 70 rows: the tensor-core tiles, ragged last tile
    (40, 7, 29, "0", "q8_0")])
def test_experts_with_shared_rows(n, begin, count, prefill, preset):
    # the expert-parallel entry point: routed experts on every row, shared expert on [begin, begin+count)
    old = os.environ.get("PMOE_PREFILL")
    os.environ["PMOE_PREFILL"] = prefill
    try:
        t = synth.make_layer(E=16, k=3, preset=preset, seed=21)
        blk = synth.make_block(t, DEV, max_tokens=n)
        ol = oracle_layer(t)
        x = seeded_x(n, 2048, 50 + n)
        rng = np.random.default_rng(5)
        idx = np.stack([rng.choice(16, size=3, replace=False) for _ in range(n)]).astype(np.uint32)
        idx[1, 2] = 0xFFFFFFFF
        w = rng.random((n, 3)).astype(np.float32)
        got = blk.experts_forward_batched(x.to(DEV), torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w), 3,
                                          shared_rows=(begin, count)).cpu().numpy()
        blk.status()
        want = ol.experts_forward(x.numpy(), idx, w)
        if count:
            want[begin:begin + count] += ol.shared_forward(x.numpy()[begin:begin + count])
        assert rel_l2(got, want) <= (1e-3 if prefill == "1" else 5e-4)
        # rows outside the range carry no shared part at all
        plain = blk.experts_forward_batched(x.to(DEV), torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w), 3)
        outside = np.ones(n, bool)
        outside[begin:begin + count] = False
        assert np.array_equal(got[outside], plain.cpu().numpy()[outside])
        # and the request does not leak into the next call
        assert rel_l2(blk.forward(x.to(DEV)).cpu().numpy(), ol.forward(x.numpy())[0]) <= REL_L2_TOL
        with pytest.raises(pm.PmoeError):
            blk.experts_forward_batched(x.to(DEV), torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w), 3,
                                        shared_rows=(n - 1, 2))
    finally:
        if old is None:
            del os.environ["PMOE_PREFILL"]
        else:
            os.environ["PMOE_PREFILL"] = old


@pytest.mark.parametrize("n", [1, 37, 700])
def test_router_stats(n):
    t = synth.make_layer(E=64, k=4, preset="q8_0", seed=6, shared=False, zipf=True)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, 2048, 90 + n).to(DEV)
    logits, w, idx = blk.route(x)
    idx = idx.clone()
    if n > 1:
        idx[1, 2] = 64        # an id past E does not count, but stays in the denominator
    counts, z, lb = blk.router_stats(logits, idx)
    want_counts, want_z, want_lb = oracle_layer(t).router_stats(logits.cpu().numpy(), idx.cpu().numpy())
    assert np.array_equal(counts.cpu().numpy(), want_counts.astype(np.float32))
    assert abs(float(z) - want_z) <= 1e-5 * abs(want_z)
    assert abs(float(lb) - want_lb) <= 1e-5 * abs(want_lb)
    again = blk.router_stats(logits, idx)
    assert float(again[1]) == float(z) and float(again[2]) == float(lb)   # fixed summation order


def test_expert_slices_sum_to_whole_block():
    # two expert-parallel halves of one layer give the whole layer's routed output
    t = synth.make_layer(E=64, k=6, preset="q4k_m", seed=9)
    whole = synth.make_block(t, DEV, max_tokens=32)
    lo = synth.make_block(t, DEV, max_tokens=32, expert_base=0, E_local=32)
    hi = synth.make_block(t, DEV, max_tokens=32, expert_base=32, E_local=32)
    x = seeded_x(20, 2048, 77).to(DEV)
    logits, w, idx = whole.route(x)
    full = whole.experts_forward_batched(x, idx, w)
    parts = lo.experts_forward_batched(x, idx, w) + hi.experts_forward_batched(x, idx, w)
    assert rel_l2(parts.cpu().numpy(), full.cpu().numpy()) <= 1e-6


def test_deterministic_and_host_entry_point():
    t = synth.make_layer(E=64, k=6, preset="q4k_m", seed=10)
    blk = synth.make_block(t, DEV, max_tokens=64)
    x = seeded_x(48, 2048, 4, torch.bfloat16)
    a = blk.forward(x.to(DEV)).float().cpu().numpy()
    b = blk.forward(x.to(DEV)).float().cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    out_h, (lg, idx, w) = blk.forward_host(x, with_stats=True)
    assert np.array_equal(out_h.float().numpy().view(np.uint32), a.view(np.uint32))
    ol = oracle_layer(t)
    _, want_logits, want_idx, _ = ol.forward(x.float().numpy())
    assert np.array_equal(idx.numpy().astype(np.uint32), want_idx)
    # repeated calls of one shape go through the recorded graph; another shape in between drops back
    # to direct launches; every result is the same
    x2 = seeded_x(48, 2048, 5, torch.bfloat16)
    a2 = blk.forward(x2.to(DEV)).float().cpu().numpy()
    for i in range(5):
        xi, ai = (x, a) if i % 2 == 0 else (x2, a2)
        assert np.array_equal(blk.forward_host(xi).float().numpy().view(np.uint32), ai.view(np.uint32))
    short = blk.forward_host(x[:7])
    assert np.array_equal(short.float().numpy().view(np.uint32), blk.forward(x[:7].to(DEV)).float().cpu().numpy().view(np.uint32))
    assert np.array_equal(blk.forward_host(x).float().numpy().view(np.uint32), a.view(np.uint32))
    pinned = torch.empty((48, 2048), dtype=torch.bfloat16).pin_memory()   # written by the kernel, no copy back
    for _ in range(3):
        pinned.zero_()
        blk.forward_host(x, out_host=pinned)
        assert np.array_equal(pinned.float().numpy().view(np.uint32), a.view(np.uint32))
    out_h2, (lg2, idx2, w2) = blk.forward_host(x, with_stats=True)
    assert np.array_equal(idx2.numpy(), idx.numpy()) and np.array_equal(lg2.numpy(), lg.numpy())
    blk.status()


def test_error_behaviour():
    t = synth.make_layer(E=8, k=2, preset="q4k", seed=1)
    blk = synth.make_block(t, DEV, max_tokens=4)
    with pytest.raises(pm.PmoeError) as e:
        blk.forward(seeded_x(5, 2048, 1).to(DEV))
    assert e.value.code == -5
    with pytest.raises(pm.PmoeError):
        blk.forward(seeded_x(2, 2048, 1).to(DEV).half())
    tr = synth.make_block(t, DEV, max_tokens=4, training_mode=True)
    with pytest.raises(pm.PmoeError) as e:
        tr.forward(seeded_x(2, 2048, 1).to(DEV))
    assert e.value.code == -6
    assert blk.forward(seeded_x(0, 2048, 1).to(DEV)).shape == (0, 2048)
    # a Q3_K shared expert beside Q4_K routed experts is a pairing without kernels: refused at create
    bad = synth.make_layer(E=4, k=1, preset="q4k", seed=2)
    sh = synth.make_layer(E=4, k=1, preset="q3k", seed=2)["shared"]
    bad["shared"] = sh
    with pytest.raises(pm.PmoeError) as e:
        synth.make_block(bad, DEV, max_tokens=4)
    assert e.value.code == -2


def test_add_rms_norm():
    x = seeded_x(5, 2048, 3).to(DEV)
    dl = seeded_x(5, 2048, 4).to(DEV)
    wt = (seeded_x(1, 2048, 5)[0] * 0.1 + 1).to(DEV)
    resid, y = pm.add_rms_norm(x, dl, wt, 1e-6)
    want_resid = x.cpu().numpy() + dl.cpu().numpy()
    want = po.rms_norm(want_resid, wt.cpu().numpy(), 1e-6)
    assert np.array_equal(resid.cpu().numpy(), want_resid)
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("dtype,rows,cols", [(pm.Q4_K, 64, 2048), (pm.Q6_K, 128, 512), (pm.Q8_0, 32, 1024),
                                             (pm.Q5_K, 48, 1024), (pm.Q2_K, 40, 768), (pm.Q3_K, 35, 256),
                                             (pm.Q6_K, 33, 256)])   # 210-byte rows: every other row starts 2 bytes off a word
def test_qmatmul_entry_point(dtype, rows, cols):
    rng = np.random.default_rng(11)
    w = po.quantize(dtype, (rng.standard_normal(rows * cols) * 0.02).astype(np.float32))
    x = rng.standard_normal((5, cols)).astype(np.float32)
    want = po.qmatmul(dtype, w, rows, cols, x)
    got = pm.qmatmul(pm.QTensor(w, dtype, (rows, cols)), torch.from_numpy(x).to(DEV)).cpu().numpy()
    assert rel_l2(got, want) <= 2e-6


def test_stack_with_residual_and_rms_norm():
    # benchmark configuration 4 (layer stack) in miniature: h <- h + moe(rms_norm(h)) through independently seeded layers
    # (LayerWeights::forward_with_stats, qwen3_next.rs:4273-4286; eps 1e-6, norm weight 1)
    layers = [synth.make_layer(E=16, k=2, preset="q4k_m", seed=30, layer=li) for li in range(3)]
    blocks = [synth.make_block(t, DEV, max_tokens=16) for t in layers]
    oracles = [oracle_layer(t) for t in layers]
    h0 = seeded_x(12, 2048, 8)
    resid = h0.to(DEV)
    delta = None
    for blk in blocks:
        resid, y = pm.add_rms_norm(resid, delta, None, 1e-6)
        delta = blk.forward(y)
    resid, _ = pm.add_rms_norm(resid, delta, None, 1e-6)
    want = h0.numpy().copy()
    for ol in oracles:
        want = want + ol.forward(po.rms_norm(want, None, 1e-6))[0]
    got = resid.cpu().numpy()
    # compare the MoE contribution, not the residual stream that carries the input unchanged
    assert rel_l2(got - h0.numpy(), want - h0.numpy()) <= REL_L2_TOL
    assert max_abs(got, want) <= MAX_ABS_TOL


def test_bounded_wait_reports_timeout_and_the_layer_recovers():
    """A device-side wait that runs out: one CTA of the gate/up kernel never receives its first item (the producer
    skips that copy on request), its bounded wait expires after a few polls, the kernel records PMOE_ERR_TIMEOUT in
    the layer's status word and every CTA still leaves normally.  Nothing traps or hangs; the next call is fine."""
    t = synth.make_layer(E=64, k=6, preset="q4k_m", seed=23)
    blk = synth.make_block(t, DEV, max_tokens=64)
    x = seeded_x(64, 2048, 5, torch.bfloat16).to(DEV)
    good = blk.forward(x).float().cpu()
    blk.status()
    old = {k: os.environ.get(k) for k in ("PMOE_DEBUG", "PMOE_MAX_POLLS")}
    os.environ["PMOE_DEBUG"], os.environ["PMOE_MAX_POLLS"] = "6", "64"
    try:
        blk.forward(x)
        with pytest.raises(pm.PmoeError) as e:
            blk.status()
        assert e.value.code == -7                      # PMOE_ERR_TIMEOUT
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    blk.status()                                       # the status word was cleared by the read above
    again = blk.forward(x).float().cpu()
    blk.status()
    assert torch.equal(again, good)
