"""Expert parallelism on real GPUs (needs at least two): N ranks over NCCL must reproduce the
single-GPU block.  NVLS is switched off for the run, as for every multi-rank test on shared hosts."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
    pytest.skip("needs two CUDA devices", allow_module_level=True)


@pytest.mark.parametrize("mode,placement,preset", [
    ("native_exact", "contiguous", "q4k_m"),      # pmoe_ep_forward, all-to-all-v with exact counts
    ("native_padded", "round_robin", "q4k_m"),    # ... padded counts (no host synchronisation), experts dealt round-robin
    ("native", "contiguous", "q8_0"),             # Q8_0 rows travel
    ("native_exact", "round_robin", "q4k_q6k_all"),
    ("all_to_all", "contiguous", "q4k_m"), ("all_gather", "contiguous", "q4k_m")])
def test_expert_parallel_matches_single_gpu(mode, placement, preset):
    world = 2 if torch.cuda.device_count() < 4 else 4
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_gpu_worker.py"), mode, placement, preset]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "all_ok=1" in r.stdout
