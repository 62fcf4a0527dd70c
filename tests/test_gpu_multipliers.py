"""Block-scale multipliers of the training mode on the GPU (MoeExperts::set_block_multipliers,
qwen3_next.rs:1705-1720; QTensor::modify_block_scales through build_scaled_mats, 1554-1621, and
QMatMul::forward_with_scales, models/with_tracing.rs:217-248) against the CPU oracle."""
import numpy as np
import pytest
import torch

from tests.common import MAX_ABS_TOL, REL_L2_TOL, max_abs, oracle_layer, rel_l2, seeded_x

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import paramecia_b200 as pm
from paramecia_b200 import synth
from oracle import pmoe_oracle as po

DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [pm.Q2_K, pm.Q3_K, pm.Q4_K, pm.Q5_K, pm.Q6_K, pm.Q8_0])
def test_modify_block_scales_bit_exact(dtype):
    rng = np.random.default_rng(21)
    bs, nb = pm.block_size(dtype), 4096 + 3
    w = po.quantize(dtype, (rng.standard_normal(nb * bs) * 0.02).astype(np.float32))
    m = rng.uniform(0.25, 4.0, nb).astype(np.float32)
    m[:4] = [1.0, 0.0, -2.0, 1e-3]
    want = po.modify_block_scales(dtype, w, m)
    q = pm.QTensor(torch.from_numpy(w).to(DEV), dtype, (nb, bs))
    got = pm.modify_block_scales(q, torch.from_numpy(m).to(DEV))
    assert np.array_equal(got.data.cpu().numpy(), want)


def _scaled_layer(t, mg, mu, md, sg=None, su=None, sd=None):
    """The oracle's layer with the multipliers folded into copies of the weights (what build_scaled_mats does)."""
    t2 = dict(t)
    for name, m in (("gate", mg), ("up", mu), ("down", md)):
        t2[name] = torch.from_numpy(po.modify_block_scales(t[name + "_dtype"], t[name].cpu().numpy(), m))
    if t["shared"] is not None:
        s = dict(t["shared"])
        for name, m in (("gate", sg), ("up", su), ("down", sd)):
            if m is not None:
                s[name] = torch.from_numpy(po.modify_block_scales(s[name + "_dtype"], s[name].cpu().numpy(), m))
        t2["shared"] = s
    return oracle_layer(t2)


@pytest.mark.parametrize("preset,n", [("q4k_m", 5), ("q4k", 33), ("q8_0", 9), ("q4k_q6k_all", 700)])
def test_block_with_multipliers_matches_oracle(preset, n):
    E, k = 32, 4
    t = synth.make_layer(E=E, k=k, preset=preset, seed=31)
    blk = synth.make_block(t, DEV, max_tokens=max(n, 64))
    rng = np.random.default_rng(5)
    d = blk._desc
    nb = lambda which: blk._blocks_of(which)
    mg, mu, md = (rng.uniform(0.5, 1.5, nb(w)).astype(np.float32) for w in ("gate", "up", "down"))
    sg, sd = (rng.uniform(0.5, 1.5, nb(w)).astype(np.float32) for w in ("sh_gate", "sh_down"))
    x = seeded_x(n, 2048, 17, torch.bfloat16)
    plain, _ = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.set_block_multipliers(torch.from_numpy(mg), torch.from_numpy(mu), torch.from_numpy(md))
    blk.set_shared_scales(gate_scales=torch.from_numpy(sg), down_scales=torch.from_numpy(sd))
    out, (logits, idx) = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    blk.status()
    want, want_logits, want_idx, _ = _scaled_layer(t, mg, mu, md, sg, None, sd).forward(x.float().numpy())
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), want_idx)
    got = out.cpu().numpy()
    assert rel_l2(got, want) <= REL_L2_TOL and max_abs(got, want) <= MAX_ABS_TOL
    assert rel_l2(plain.cpu().numpy(), want) > 1e-2          # the multipliers did change the result
    # the host-buffer entry point must not replay a chain recorded with the old weights
    xh = x.clone()
    for _ in range(4):
        oh = blk.forward_host(xh)
    assert rel_l2(oh.float().numpy(), want) <= 5e-3          # bf16 output
    blk.clear_block_multipliers()
    blk.set_shared_scales()
    for _ in range(2):
        oh = blk.forward_host(xh)
    again, _ = blk.forward_with_stats(x.to(DEV), out_dtype=torch.float32)
    assert torch.equal(again, plain)
    assert rel_l2(oh.float().numpy(), plain.cpu().numpy()) <= 5e-3


def test_multiplier_argument_checks():
    t = synth.make_layer(E=8, k=2, preset="q4k", seed=1)
    blk = synth.make_block(t, DEV, max_tokens=8)
    g = torch.ones(blk._blocks_of("gate"))
    with pytest.raises(ValueError):
        blk.set_block_multipliers(g[:-1], g, torch.ones(blk._blocks_of("down")))
    lib = pm.lib()
    rc = lib.pmoe_layer_set_block_multipliers(blk._h, g.to(DEV).data_ptr(), None, None, None)
    assert rc == -1 and b"together" in lib.pmoe_last_error()
