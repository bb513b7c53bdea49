"""The "eccl" process group on real devices. World size 1 runs everywhere; the
world-size-2 run needs two GPUs and is skipped otherwise. Failure handling is
exercised on the host only: no test makes a GPU fault or hang."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "eccl_worker.py"), str(r), str(world)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    assert "ECCL_OK" in outs[0]


def test_eccl_world_size_1():
    _run(1, 29711)


def test_eccl_world_size_2():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, 29712)


def test_eccl_world_size_4():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    _run(4, 29713)
