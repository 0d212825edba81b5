"""GPU, two or more devices: tensor-parallel shards (heads and FFN columns per rank; attention output and FFN activation
all-gathered, Wo and W_down replicated) against the single-GPU result, bit for bit - with the exchange fused into the
kernels over peer memory and with NCCL all-gathers, on a small model and on a deep one. Skipped on a one-GPU box."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("model", ["small", "deep"])
@pytest.mark.parametrize("nccl_only", [False, True])
@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_matches_single_gpu(world, nccl_only, model, tmp_path):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "tp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if nccl_only:
        env["SPYB_TP_NCCL_ONLY"] = "1"   # NCCL all-gathers for every step (else: the exchange fused into the kernels)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29541", worker, str(tmp_path / "tp.gguf"), model]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0 and "OK" in r.stdout
