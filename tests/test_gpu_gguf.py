"""GGUF ingestion on the GPU: a block loaded from a GGUF file equals the block built from the same tensors
in memory, for whole layers, expert-parallel slices and 16-bit router weights."""
import numpy as np
import pytest
import torch

from tests.common import REL_L2_TOL, oracle_layer, rel_l2, seeded_x

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

gguf = pytest.importorskip("gguf")

from paramecia_b200 import synth
from paramecia_b200.gguf import GGUFError, GGUFFile, load_moe_block
from tests.gguf_util import write_layer_gguf

DEV = "cuda:0"


@pytest.mark.parametrize("preset,alt", [("q4k_m", False), ("q4k_q6k_all", True)])
def test_block_from_gguf_equals_block_from_memory(tmp_path, preset, alt):
    t = synth.make_layer(E=16, k=3, preset=preset, seed=31)
    path = str(tmp_path / "l.gguf")
    write_layer_gguf(path, t, layer=2, alt_gate_name=alt)
    x = seeded_x(12, 2048, 4, torch.bfloat16).to(DEV)
    direct = synth.make_block(t, DEV, max_tokens=16)
    with GGUFFile(path) as f:
        blk = load_moe_block(f, 2, DEV, max_tokens=16)
        assert blk.num_experts == 16 and blk.num_experts_per_tok == 3 and blk.has_shared
        out, (logits, idx) = blk.forward_with_stats(x, out_dtype=torch.float32)
        want, (wl, wi) = direct.forward_with_stats(x, out_dtype=torch.float32)
        assert torch.equal(out, want) and torch.equal(logits, wl) and torch.equal(idx, wi)
        ref = oracle_layer(t).forward(x.float().cpu().numpy())[0]
        assert rel_l2(out.cpu().numpy(), ref) <= REL_L2_TOL
        with pytest.raises(GGUFError):
            load_moe_block(f, 3, DEV)


def test_expert_parallel_slices_from_gguf(tmp_path):
    t = synth.make_layer(E=16, k=4, preset="q4k_m", seed=32)
    path = str(tmp_path / "l.gguf")
    write_layer_gguf(path, t)
    x = seeded_x(9, 2048, 5).to(DEV)
    with GGUFFile(path) as f:
        whole = load_moe_block(f, 0, DEV, max_tokens=16)
        parts = [load_moe_block(f, 0, DEV, max_tokens=16, ep_rank=r, ep_size=4) for r in range(4)]
    logits, w, idx = whole.route(x)
    full = whole.experts_forward_batched(x, idx, w)
    acc = sum(p.experts_forward_batched(x, idx, w) for p in parts)
    assert parts[1].expert_base == 4 and parts[1].num_experts_local == 4
    assert rel_l2(acc.cpu().numpy(), full.cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("router", ["f16", "bf16"])
def test_sixteen_bit_router_weights(tmp_path, router):
    # the library widens them once; the logits must equal those of the widened f32 weights bit for bit
    t = synth.make_layer(E=32, k=4, preset="q8_0", seed=33, shared=False)
    path = str(tmp_path / "l.gguf")
    write_layer_gguf(path, t, router_dtype=router)
    dt = torch.float16 if router == "f16" else torch.bfloat16
    t_wide = dict(t, router_w=t["router_w"].to(dt).float())
    x = seeded_x(20, 2048, 6).to(DEV)
    with GGUFFile(path) as f:
        blk = load_moe_block(f, 0, DEV, max_tokens=32)
    logits, w, idx = blk.route(x)
    ol = oracle_layer(t_wide)
    want = ol.router_logits(x.cpu().numpy())
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), ol.route_topk(want)[0])


def test_quantised_router_from_gguf(tmp_path):
    # a GGUF whose ffn_gate_inp is Q8_0 blocks: the router runs as a quantised mat-mul, as the reference's QMatMul does
    t = synth.make_layer(E=32, k=4, preset="q4k_m", seed=34, router_dtype=8)
    path = str(tmp_path / "l.gguf")
    write_layer_gguf(path, t, router_dtype="blocks")
    x = seeded_x(20, 2048, 7).to(DEV)
    with GGUFFile(path) as f:
        blk = load_moe_block(f, 0, DEV, max_tokens=32)
    direct = synth.make_block(t, DEV, max_tokens=32)
    out, (logits, idx) = blk.forward_with_stats(x, out_dtype=torch.float32)
    want, (wl, wi) = direct.forward_with_stats(x, out_dtype=torch.float32)
    assert torch.equal(out, want) and torch.equal(logits, wl) and torch.equal(idx, wi)
    ref = oracle_layer(t).forward(x.cpu().numpy())
    assert np.allclose(logits.cpu().numpy(), ref[1], rtol=1e-5, atol=1e-6)
    assert rel_l2(out.cpu().numpy(), ref[0]) <= REL_L2_TOL
