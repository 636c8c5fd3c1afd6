"""Tensor parallelism: host-side logic on two gloo ranks (CPU), and the decoder on two GPUs over NCCL."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _launch(mode, nproc):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "tp_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)


def test_two_gloo_ranks_on_cpu():
    res = _launch("cpu", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert res.stdout.count("cpu ok") == 2


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    res = _launch("watch", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "saw rank 1 leave" in res.stdout and "left after three steps" in res.stdout


@pytest.mark.gpu
def test_decoder_on_two_gpus():
    from nn_b200.device import Device
    if Device.count() < 2:
        pytest.skip("needs two GPUs")
    res = _launch("gpu", 2)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert res.stdout.count("gpu ok") == 2
