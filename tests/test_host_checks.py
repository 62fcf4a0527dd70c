"""Host-side argument checks of the Python binding: a caller-owned buffer reaches the C ABI as a raw pointer, so its
dtype, shape, device and contiguity are checked before the pointer is taken (a wrong buffer would otherwise be read
or written out of bounds on the device)."""
import pytest
import torch

import paramecia_b200 as pm
from paramecia_b200.moe import _check_buffer


def test_check_buffer_rules():
    ok = torch.zeros((4, 8), dtype=torch.float32)
    _check_buffer("x", ok, (4, 8), torch.float32, "cpu")
    _check_buffer("x", ok, (4, 8), (torch.float32, torch.bfloat16), "cpu")
    with pytest.raises(ValueError, match="float32"):
        _check_buffer("x", ok.to(torch.bfloat16), (4, 8), torch.float32, "cpu")
    with pytest.raises(ValueError, match="shape"):
        _check_buffer("x", ok, (4, 9), torch.float32, "cpu")
    with pytest.raises(ValueError, match="contiguous"):
        _check_buffer("x", torch.zeros((8, 4)).t(), (4, 8), torch.float32, "cpu")
    with pytest.raises(ValueError, match="must live on"):
        _check_buffer("x", ok, (4, 8), torch.float32, "cuda:0")
    with pytest.raises(ValueError, match="torch tensor"):
        _check_buffer("x", [1, 2], (2,), torch.float32, "cpu")


def test_noalloc_matmul_refuses_host_and_mistyped_buffers():
    w = pm.QTensor(torch.zeros(144 * 8, dtype=torch.uint8), pm.Q4_K, (8, 256))
    x = torch.zeros((2, 256))
    y = torch.zeros((2, 8))
    with pytest.raises(ValueError):
        pm.qmatmul_noalloc(w, x, y)   # host tensors: nothing may be copied behind the caller's back


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")
def test_entry_points_refuse_wrong_buffers_on_the_gpu():
    from paramecia_b200 import synth
    dev = "cuda:0"
    t = synth.make_layer(E=8, k=2, preset="q4k", seed=1)
    blk = synth.make_block(t, dev, max_tokens=8)
    x = torch.zeros((4, 2048), dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):
        blk.forward_into(x, torch.zeros((3, 2048), dtype=torch.bfloat16, device=dev))      # too few rows
    with pytest.raises(ValueError):
        blk.forward_into(x.half(), torch.zeros((4, 2048), dtype=torch.bfloat16, device=dev))  # f16 is not served
    with pytest.raises(ValueError):
        blk.forward_into(x, torch.zeros((4, 4096), dtype=torch.bfloat16, device=dev)[:, ::2])  # strided
    with pytest.raises(ValueError):
        blk.route(x, out=(torch.zeros((4, 8), device=dev), torch.zeros((4, 2), device=dev),
                          torch.zeros((4, 2), dtype=torch.int64, device=dev)))              # ids must be int32
    with pytest.raises(ValueError):
        blk.experts_forward_batched(x, torch.zeros((4, 2), dtype=torch.int32), torch.zeros((4, 2)), 2,
                                    out=torch.zeros((4, 2048), dtype=torch.float16, device=dev))
    w = pm.QTensor(t["gate"][:144 * 8 * 8].to(dev), pm.Q4_K, (8, 2048))
    xf = torch.zeros((2, 2048), device=dev)
    with pytest.raises(ValueError):
        pm.qmatmul_noalloc(w, xf.to(torch.bfloat16), torch.zeros((2, 8), device=dev))       # bf16 x would be read as f32
    with pytest.raises(ValueError):
        pm.qmatmul_noalloc(w, xf, torch.zeros((2, 4), device=dev))                          # y too small
    pm.qmatmul_noalloc(w, xf, torch.zeros((2, 8), device=dev))
