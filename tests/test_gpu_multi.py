"""Vocabulary-parallel lm_head on real GPUs (needs at least two; skipped otherwise):
one rank per GPU under torch.distributed.run, NCCL for the all-gather form, CUDA IPC
peer memory for the exchange inside the kernel.  The single-GPU suite covers the same
kernels with both ranks' buffers on one device (tests/test_gpu_parity.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4])
def test_vocabulary_parallel_pick_equals_oracle(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world),
           os.path.join(HERE, "vocab_parallel_gpu_worker.py")]
    out = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-4000:]
    assert f"on {world} GPUs: ok" in out.stdout
