"""Multi-GPU check of the partitioned convolution (NCCL halo exchange overlapped with the interior
rows + the native kernels): the rows every rank owns must equal the same rows of the single-GPU
convolution bit for bit.  Runs on 2 GPUs, and on 4 where that many are visible; skipped with fewer."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world,port", [(2, 29561), (4, 29563)])
def test_partitioned_conv_matches_single_gpu(world, port):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(port), "-m", "warpconvnet_b200.examples.partitioned_conv_bench",
           "--voxels", "300000", "--sweeps", "4", "--azimuth-steps", "2048", "--channels", "64", "--dtype", "bf16",
           "--iters", "2", "--check"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["n_gpus"] == world and out["halo_rows_total"] > 0 and out["boundary_rows_total"] > 0
    assert out["max_abs_diff_vs_single_gpu"] == 0.0
