"""Expert-parallel layer on 2 (or 4) GPUs of one box: NCCL all-to-all-v dispatch and combine around
the grouped GEMMs, each rank checked against the CPU oracle.  Skipped on a single-GPU box."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,passes,exchange", [(2, 1, "nccl"), (2, 2, "nccl"), (2, 2, "push"), (2, 1, "fused"),
                                                   (4, 1, "nccl"), (4, 4, "push"), (4, 1, "fused"), (8, 1, "fused"),
                                                   (2, 1, "allreduce"), (4, 1, "allreduce"),
                                                   (2, 1, "allreduce-int8"), (4, 1, "allreduce-fp8")])
def test_ep_layer_matches_oracle(world, passes, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ar_quant = exchange.partition("-")[2]                # quantized all-reduce payload of the all-reduce strategy
    exchange = exchange.partition("-")[0]
    port = (29600 + os.getpid() % 300 + 10 * world + passes + {"nccl": 0, "push": 5, "fused": 7, "allreduce": 8}[exchange]
            + (3 if ar_quant else 0))
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", EP_PASSES=str(passes),
                   EP_EXCHANGE="auto" if exchange == "allreduce" else exchange,
                   EP_STRATEGY="allreduce" if exchange == "allreduce" else "all2all", EP_AR_QUANT=ar_quant)
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "ep_worker.py"), ROOT], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out))
    for rc, out in outs:
        assert rc == 0, out[-3000:]
