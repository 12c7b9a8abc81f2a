"""Tensor-parallel decode across GPUs of one node (needs at least two GPUs; skipped otherwise)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.parametrize("kind,batch", [("llama", 2), ("deepseek", 2), ("llama", 1)])
def test_sharded_decode_matches_oracle(kind, batch):
    n = gpu_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n >= 4 else 2
    # the worker lowers the large-message threshold (deepj_cuda_tp_configure) so that the prompt chunks' exchanges
    # (24576 values) take the chunk-sized grid and the decode steps' the small one
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29621", os.path.join(HERE, "tp_gpu_worker.py"), kind, str(batch)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and "TP_GPU_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
