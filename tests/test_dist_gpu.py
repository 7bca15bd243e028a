"""ShardedDecoder on real ranks: one process per GPU under torchrun (needs at least two GPUs; the single-GPU run of the
suite covers the same kernel with all ranks played in one cooperative launch, tests/test_fmha_gpu.py)."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_decoder_on_real_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this machine has {torch.cuda.device_count()}")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")  # the exchange uses plain peer stores; NCCL only sets up and checks
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert r.returncode == 0 and len(lines) == world and all(x["ok"] for x in lines), (r.stdout[-3000:], r.stderr[-3000:])
