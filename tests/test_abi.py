"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/pmoe.h declares; without a device it refuses to create a layer instead of
computing anything on the CPU."""
import ctypes as C
import os
import re

import pytest
import torch

import paramecia_b200 as pm
from paramecia_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "pmoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pmoe_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert "pmoe_forward" in names and "pmoe_layer_create" in names and len(names) >= 15
    raw = C.CDLL(pm.lib_path())
    bound = {n for n, _, _ in _lib.SYMBOLS}
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in pmoe.h but not exported by libpmoe.so"
        assert n in bound, f"{n} has no ctypes binding"


def test_sizes_and_version():
    assert pm.lib().pmoe_version() == 4
    assert (pm.block_size(pm.Q4_K), pm.type_size(pm.Q4_K)) == (256, 144)
    assert (pm.block_size(pm.Q6_K), pm.type_size(pm.Q6_K)) == (256, 210)
    assert (pm.block_size(pm.Q8_0), pm.type_size(pm.Q8_0)) == (32, 34)
    assert pm.row_bytes(pm.Q4_K, 2048) == 1152 and pm.row_bytes(pm.Q6_K, 512) == 420
    assert pm.block_size(99) == 0


def test_descriptor_validation_needs_no_gpu():
    d = _lib.LayerDesc()
    h = C.c_void_p()
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -1       # wrong struct_size
    assert b"struct_size" in pm.lib().pmoe_last_error()
    d.struct_size = C.sizeof(_lib.LayerDesc)
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -1       # zero shapes
    d.H, d.F, d.E, d.k, d.max_tokens = 2048, 512, 8, 2, 4
    d.gate_dtype = d.up_dtype = d.down_dtype = 2                            # Q4_0: not served
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -2
    d.gate_dtype, d.up_dtype, d.down_dtype = pm.Q4_K, pm.Q6_K, pm.Q6_K
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -2       # gate and up must match
    d.up_dtype = pm.Q4_K
    d.H = 1024
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -3       # shape not served
    assert h.value is None


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU refusal")
def test_no_cpu_fallback():
    from paramecia_b200 import synth
    t = synth.make_layer(E=4, k=1, preset="q4k", seed=0)
    with pytest.raises(pm.PmoeError) as e:
        synth.make_block(t, "cpu")
    assert e.value.code == -9
    d = _lib.LayerDesc()
    d.struct_size = C.sizeof(_lib.LayerDesc)
    d.H, d.F, d.E, d.k, d.max_tokens = 2048, 512, 4, 1, 4
    d.gate_dtype = d.up_dtype = d.down_dtype = pm.Q4_K
    h = C.c_void_p()
    assert pm.lib().pmoe_layer_create(C.byref(d), C.byref(h)) == -9
    assert b"no CPU path" in pm.lib().pmoe_last_error()
    assert pm.lib().pmoe_forward(None, None, 0, 1, None, 0, None, None, None, None) == -1
