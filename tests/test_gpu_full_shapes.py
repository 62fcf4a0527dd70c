"""GPU parity against the CPU oracle at the benchmark configurations' real sizes: 512 experts,
top-10, hidden 2048, intermediate 512 -- the shapes the benchmark itself runs, not miniatures.

* prefill of 4096 bf16 tokens with the Zipf-biased router (configuration 3), path chosen by the
  library itself (token-sorted grouped tcgen05 GEMMs);
* the all-Q8_0 block over thousands of tokens (the class of configuration 5);
* the call one expert-parallel rank of eight makes: 512 received rows, 64 local experts, the
  shared expert on the rank's own 64 rows.

Bars: top-k indices equal, max-abs 2e-2 and relative-L2 1e-3 against the oracle.
"""
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
H, F, E, K = 2048, 512, 512, 10


@pytest.mark.parametrize("preset", ["q4k_q6k_all", "q4k_m"])
def test_prefill_4096_tokens_zipf_routing(preset):
    n = 4096
    t = synth.make_layer(H, F, E, K, preset, seed=31, device=DEV, zipf=True)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, H, 71, torch.bfloat16)
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    ol = oracle_layer(t)
    want, want_logits, want_idx, _ = ol.forward(x.float().numpy())
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want_logits.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    counts = np.bincount(want_idx.ravel(), minlength=E)
    assert counts.max() >= n // 2 and (counts == 0).sum() > E // 2   # a few experts take most tokens
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(got, want) <= REL_L2_TOL


def test_q8_0_block_2048_tokens_zipf_routing():
    n = 2048
    t = synth.make_layer(H, F, E, K, "q8_0", seed=32, device=DEV, zipf=True)
    blk = synth.make_block(t, DEV, max_tokens=n)
    x = seeded_x(n, H, 72, torch.bfloat16)
    out, (_, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    want, _, want_idx, _ = oracle_layer(t).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("rank", [0, 5])
def test_one_rank_of_eight(rank):
    # what rank `rank` of eight computes in the 8-GPU benchmark: 8 x 64 rows arrive, the rank owns
    # experts [64*rank, 64*rank + 64) and is home to rows [64*rank, 64*rank + 64)
    world, n_home = 8, 64
    rows, El = world * n_home, E // world
    t = synth.make_layer(H, F, E, K, "q4k_m", seed=33, device=DEV)
    whole = synth.make_block(t, DEV, max_tokens=rows)
    part = synth.make_block(t, DEV, max_tokens=rows, expert_base=rank * El, E_local=El)
    x = seeded_x(rows, H, 73, torch.bfloat16).to(DEV)
    _, w, idx = whole.route(x)
    got = part.experts_forward_batched(x, idx, w, K, shared_rows=(rank * n_home, n_home),
                                       out_dtype=torch.float32).cpu().numpy()
    part.status()
    ol = oracle_layer(t)
    ids = idx.cpu().numpy().astype(np.int64)
    mine = np.where((ids >= rank * El) & (ids < (rank + 1) * El), ids, 0xFFFFFFFF).astype(np.uint32)
    xf = x.float().cpu().numpy()
    want = ol.experts_forward(xf, mine, w.cpu().numpy())
    own = slice(rank * n_home, (rank + 1) * n_home)
    want[own] += ol.shared_forward(xf[own])
    assert max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(got, want) <= REL_L2_TOL
    # the eight slices add up to the whole block's output on every row
    if rank == 0:
        total = torch.zeros((rows, H), dtype=torch.float32, device=DEV)
        for r in range(world):
            blk_r = part if r == rank else synth.make_block(t, DEV, max_tokens=rows, expert_base=r * El, E_local=El)
            total += blk_r.experts_forward_batched(x, idx, w, K, shared_rows=(r * n_home, n_home), out_dtype=torch.float32)
        full = whole.forward(x).float()
        assert rel_l2(total.cpu().numpy(), full.cpu().numpy()) <= 3e-3   # bf16 rounding of `full`
