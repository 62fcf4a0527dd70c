"""The allocation-free quantised mat-mul entry point (pmoe_qmatmul_noalloc) against the ordinary one.

Some hosts may not allocate device memory once they are running (all of it already belongs to
their own pool, or allocator calls are banned on the request path).  For them the library keeps
the quantised activations in a fixed built-in buffer.  This file checks, through the C ABI, that
two calls in a row give exactly what pmoe_qmatmul gives, that the second call is not disturbed by
what the first left in the shared buffer, and that operands too large for the buffer are refused
with a clear message instead of being truncated.  It is named to be collected last.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import paramecia_b200 as pm
from oracle import pmoe_oracle as po

DEV = "cuda:0"


def _case(dtype, rows, cols, m, seed):
    rng = np.random.default_rng(seed)
    w = po.quantize(dtype, (rng.standard_normal(rows * cols) * 0.02).astype(np.float32))
    qt = pm.QTensor(torch.from_numpy(w).to(DEV), dtype, (rows, cols))
    x = torch.from_numpy(rng.standard_normal((m, cols)).astype(np.float32)).to(DEV)
    return qt, x


def test_two_calls_match_the_allocating_entry_point():
    # different dtypes, shapes and row counts back to back: the second call reuses the same
    # built-in buffer, which still holds the first call's quantised rows
    a_w, a_x = _case(pm.Q4_K, 96, 2048, 24, 1)
    b_w, b_x = _case(pm.Q8_0, 64, 512, 7, 2)
    a_y = torch.full((24, 96), float("nan"), device=DEV)
    b_y = torch.full((7, 64), float("nan"), device=DEV)
    pm.qmatmul_noalloc(a_w, a_x, a_y)      # the first call on the device also looks up the buffer's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    pm.qmatmul_noalloc(a_w, a_x, a_y)
    pm.qmatmul_noalloc(b_w, b_x, b_y)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before       # the calls took no device memory (the driver's own count)
    want_a = pm.qmatmul(a_w, a_x)
    want_b = pm.qmatmul(b_w, b_x)
    # same kernels, same arithmetic, only the scratch differs: bit-identical (tolerance 0)
    assert torch.equal(a_y, want_a)
    assert torch.equal(b_y, want_b)
    # and once more in the other order
    pm.qmatmul_noalloc(a_w, a_x, a_y.zero_())
    torch.cuda.synchronize()
    assert torch.equal(a_y, want_a)
    # the oracle agrees within the tolerance used for the allocating entry point
    ref = po.qmatmul(pm.Q4_K, a_w.data.cpu().numpy(), 96, 2048, a_x.cpu().numpy())
    assert np.linalg.norm(a_y.cpu().numpy() - ref) / np.linalg.norm(ref) <= 2e-6


def test_oversized_operands_are_refused():
    w, x = _case(pm.Q6_K, 32, 2048, 64, 3)   # 64 rows of 2048 do not fit the 96 KB buffer
    y = torch.empty((64, 32), device=DEV)
    with pytest.raises(pm.PmoeError) as e:
        pm.qmatmul_noalloc(w, x, y)
    assert e.value.code == -5 and "built-in buffer" in e.value.message
    # the largest operands that fit, and the first that do not
    w, x = _case(pm.Q8_0, 16, 2048, 39, 4)
    pm.qmatmul_noalloc(w, x[:38].contiguous(), torch.empty((38, 16), device=DEV))
    with pytest.raises(pm.PmoeError):
        pm.qmatmul_noalloc(w, x, torch.empty((39, 16), device=DEV))
    # the column limit of pmoe_qmatmul holds here too
    lib = pm.lib()
    rc = lib.pmoe_qmatmul_noalloc(0, pm.Q8_0, w.data.data_ptr(), 1, 32768, x.data_ptr(), 1, x.data_ptr(), None)
    assert rc == -3
