"""Multi-GPU tests: run the worker under torch.distributed.run on 2 GPUs (skipped with fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode: str, nproc: int = 2, port: int = 29631, nvls: bool = True):
    if not torch.cuda.is_available() or torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    # NCCL's own NVLS stays off in the tests; this library's switch-multicast path is on unless the test is
    # one in which a rank is late or leaves (those run on plain peer memory)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", FLODL_B200_NVLS="1" if nvls else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mg_worker.py"), mode]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and f"MG_OK {mode}" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


def test_symmetric_collectives_2gpu():
    _run("collectives", 2, 29631)


def test_symm_collectives_4gpu():
    _run("collectives", 4, 29641)


def test_symmetric_collectives_peer_path_2gpu():
    _run("collectives", 2, 29638, nvls=False)


def test_symm_collectives_3gpu_odd_world():
    _run("collectives", 3, 29643)


def test_late_rank_never_applies_unreduced_gradients_2gpu():
    _run("giveup", 2, 29639, nvls=False)


def test_train_engine_ddp_4gpu():
    _run("engine", 4, 29642)


def test_train_engine_ddp_2gpu():
    _run("engine", 2, 29632)


def test_engine_broadcasts_batchnorm_buffers_2gpu():
    _run("resnet_buffers", 2, 29633)


def test_graph_ddp_trainer_setup_2gpu():
    _run("graph_ddp", 2, 29634)


@pytest.mark.parametrize("mode,port", [("async_fixed", 29635), ("async_cadence", 29636), ("async_cpu", 29637)])
def test_async_ddp_2gpu(mode, port):
    _run(mode, 2, port)
