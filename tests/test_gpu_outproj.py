"""Row-parallel out-projection with the reduce-scatter in the GEMM epilogue:
as a group of one on a single GPU, and across 2 / 4 / 8 GPUs when the box has
them (one process per GPU, NVLS off, plain peer stores)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [1, 2, 4, 8])
def test_outproj_residual_across_gpus(nproc):
    import torch
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % nproc,
                          "--master-addr", "127.0.0.1", "--master-port", "29441",
                          os.path.join(ROOT, "tests", "outproj_gpu_worker.py")],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "OUTPROJ_OK" in out.stdout, out.stdout[-3000:]
