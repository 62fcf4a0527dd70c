"""paramecia_b200 -- host-side binding of libpmoe, the B200 (sm_100a) implementation of
paramecia's Qwen3-Next quantised mixture-of-experts FFN block.

The package mirrors the reference's interface for this path (``MoeBlock``, ``MoeExperts``,
``SharedExpert``, ``QTensor`` in paramecia-model/src/qwen3_next.rs and
``topk_moe_routing`` in paramecia-model/src/ops.rs) on top of the C ABI declared in
``include/pmoe.h``.  PyTorch supplies device memory, streams and ``torch.distributed``;
all arithmetic of the block runs in the library's CUDA kernels.  There is no CPU path: the
import fails if ``libpmoe.so`` has not been built, and constructing a layer fails without a GPU.
"""
from ._lib import (PmoeError, lib, lib_path, launch_count, F32, F16, BF16, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K,
                   block_size, type_size, row_bytes)
from .moe import QTensor, MoeBlock, SharedExpertWeights, dequantize, add_rms_norm, add_rms_norm_into, qmatmul, qmatmul_noalloc, modify_block_scales
from .gguf import GGUFFile, GGUFError, load_moe_block, moe_layers

__all__ = ["PmoeError", "lib", "lib_path", "launch_count", "F32", "F16", "BF16", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K",
           "block_size", "type_size", "row_bytes", "QTensor", "MoeBlock", "SharedExpertWeights",
           "dequantize", "add_rms_norm", "add_rms_norm_into", "qmatmul", "qmatmul_noalloc", "modify_block_scales", "GGUFFile", "GGUFError", "load_moe_block",
           "moe_layers"]
