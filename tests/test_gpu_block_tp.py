"""Tensor-parallel single-stream block on several GPUs (one process per GPU):
the all-gather inside the LayerNorm's stores and the input projection's
arrival waits, the reduce-scatter inside the output projection's epilogue."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_worker(nproc, mode, port):
    import torch
    if torch.cuda.device_count() < nproc:
        pytest.skip("needs %d GPUs" % nproc)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % nproc,
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "tests", "tp_block_gpu_worker.py"), mode],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "TP_OK" in out.stdout, out.stdout[-3000:]


@pytest.mark.parametrize("nproc", [1, 2, 4, 8])
def test_tensor_parallel_block(nproc):
    """Small shapes, even and uneven rows, three blocks in a row; a group of
    one runs the same kernels (stores to itself) on a single GPU."""
    run_worker(nproc, "toy", 29461)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_tensor_parallel_block_at_klein4b_widths(nproc):
    run_worker(nproc, "klein4b", 29463)
