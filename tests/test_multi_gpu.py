"""Expert / tensor / vocabulary-parallel granite step on 2 GPUs against the single-GPU step (needs >= 2 GPUs)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2])
def test_sharded_granite_matches_single_gpu(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = Path(__file__).parent / "multi_gpu_granite.py"
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29617", str(script)],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "MULTI_GPU_OK" in run.stdout, run.stdout[-2000:] + run.stderr[-3000:]


@pytest.mark.parametrize("world", [2])
def test_sharded_qwen3_5_matches_single_gpu(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = Path(__file__).parent / "multi_gpu_qwen35.py"
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29619", str(script)],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "MULTI_GPU_OK" in run.stdout, run.stdout[-2000:] + run.stderr[-3000:]
