"""GPU parity of the prefill path (tcgen05 grouped GEMMs) against the CPU oracle.

Gate/up run as exact integer block sums on the tensor cores, so silu(gate)*up matches the oracle
to f32 rounding; the down projection uses fp16 operands, which puts the block output about 3e-4
(relative L2) from the oracle -- inside the bar of max-abs 2e-2 / relative-L2 1e-3."""
import os

import numpy as np
import pytest
import torch

from tests.common import MAX_ABS_TOL, REL_L2_TOL, max_abs, oracle_layer, rel_l2, seeded_x

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import paramecia_b200 as pm
from paramecia_b200 import synth

DEV = "cuda:0"


@pytest.fixture
def force_prefill():
    old = os.environ.get("PMOE_PREFILL")
    os.environ["PMOE_PREFILL"] = "1"
    yield
    if old is None:
        del os.environ["PMOE_PREFILL"]
    else:
        os.environ["PMOE_PREFILL"] = old


@pytest.mark.parametrize("preset,E,k,n", [("q4k", 8, 2, 200), ("q4k_q6k_all", 16, 3, 333), ("q4k_q6k_all", 4, 1, 65),
                                          ("q8_0", 8, 2, 200), ("q8_0", 4, 1, 65), ("q4k_m", 16, 3, 333)])
def test_forced_prefill_matches_oracle(force_prefill, preset, E, k, n):
    t = synth.make_layer(E=E, k=k, preset=preset, seed=13)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, 2048, 40 + n, torch.bfloat16)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    want, want_logits, want_idx, _ = oracle_layer(t).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(got, want) <= REL_L2_TOL
    assert rel_l2(got, want) <= 6e-4   # fp16 down GEMM: expected about 3e-4


@pytest.mark.parametrize("prefill", ["0", "1"])
def test_grouping_spread_over_ctas(prefill):
    # 1100 tokens x top-8 = 8800 (token, slot) pairs: from 8192 pairs on the counting and the scatter of the
    # grouping run one CTA per 1024 pairs (here nine, the last one ragged) around the one-CTA scan; both the
    # tensor-core kernels and the streaming ones read its lists
    n = 1100
    old = os.environ.get("PMOE_PREFILL")
    os.environ["PMOE_PREFILL"] = prefill
    try:
        t = synth.make_layer(E=64, k=8, preset="q4k_q6k_all", seed=17, zipf=True)
        blk = synth.make_block(t, DEV, max_tokens=n)
        x = seeded_x(n, 2048, 77, torch.bfloat16)
        out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
        blk.status()
    finally:
        if old is None:
            del os.environ["PMOE_PREFILL"]
        else:
            os.environ["PMOE_PREFILL"] = old
    want, _, want_idx, _ = oracle_layer(t).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL and rel_l2(got, want) <= REL_L2_TOL


def test_skewed_routing_takes_the_prefill_path_by_itself():
    # Zipf-biased router: a few experts get most tokens, some get none, tiles are ragged
    n = 700
    t = synth.make_layer(E=32, k=4, preset="q4k_q6k_all", seed=14, zipf=True)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, 2048, 9, torch.bfloat16)
    blk.trace(True)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    phases = blk.trace_read()
    blk.trace(False)
    blk.status()
    want, _, want_idx, _ = oracle_layer(t).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    counts = np.bincount(want_idx.ravel(), minlength=32)
    assert counts.max() > 10 * max(1, counts[counts > 0].min())   # the load really is skewed
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL and rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("preset", ["q4k", "q8_0"])
def test_prefill_equals_decode_kernels_on_gate_up(force_prefill, preset):
    # same layer through both paths: the activated rows are integer-exact in both, so the
    # outputs differ only by the fp16 down GEMM
    t = synth.make_layer(E=8, k=2, preset=preset, seed=15)
    blk = synth.make_block(t, DEV, max_tokens=128)
    x = seeded_x(128, 2048, 3, torch.bfloat16).to(DEV)
    a = blk.forward(x).float().cpu().numpy()
    os.environ["PMOE_PREFILL"] = "0"
    b = blk.forward(x).float().cpu().numpy()
    os.environ["PMOE_PREFILL"] = "1"
    assert rel_l2(a, b) <= 2e-3   # bf16 output rounding dominates here


@pytest.mark.parametrize("preset", ["q8_0", "q4k_m"])
def test_prefill_sized_call_with_a_q8_0_shared_expert(preset):
    # benchmark configuration 5 in miniature (all-Q8_0 block, Zipf routing, hundreds of tokens): Q8_0 gate/up and
    # down have tensor-core kernels of their own (one block of 32 per MMA, scales applied per block); with Q4_K
    # routed experts (q4k_m) the routed part and the Q8_0 shared expert take one launch each
    n = 600
    t = synth.make_layer(E=32, k=4, preset=preset, seed=16, zipf=True)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, 2048, 21, torch.bfloat16)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    want, _, want_idx, _ = oracle_layer(t).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL and rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("preset,mult", [("q4k_q6k_all", 3000.0), ("q8_0", 800.0)])
def test_activations_beyond_the_fp16_range(force_prefill, preset, mult):
    # silu(gate) * up far above 65504: the fp16 down GEMM sees such a row divided by a power of two and the factor
    # comes back when the accumulators are drained, so the result stays finite and within the relative bar
    n = 130
    t = synth.make_layer(E=8, k=2, preset=preset, seed=19)
    blk = synth.make_block(t, DEV, max_tokens=n)
    # (Q8_0 keeps its block scales as f16, so the reference itself overflows a little further up: smaller factor)
    x = seeded_x(n, 2048, 77) * mult
    out, (_, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    want, _, want_idx, _ = oracle_layer(t).forward(x.numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert np.isfinite(got).all() and np.abs(want).max() > 65504.0
    assert rel_l2(got, want) <= REL_L2_TOL
