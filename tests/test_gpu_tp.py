"""GPU, two or more devices: tensor-parallel shards (heads and FFN columns per rank, NCCL all-reduce after
attention-out and FFN-down) against the single-GPU result. Skipped on a one-GPU box."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nccl_only", [False, True])
@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_matches_single_gpu(world, nccl_only, tmp_path):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "tp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if nccl_only:
        env["SPYB_TP_NCCL_ONLY"] = "1"   # all-reduce through NCCL for every step (else: fused peer-memory exchange for decode)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29541", worker, str(tmp_path / "tp.gguf")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0 and "OK" in r.stdout
