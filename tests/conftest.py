"""pytest configuration: the `gpu` marker and shared fixtures.

Tests marked `gpu` call libns_b200.so through its C ABI on a real B200 and compare with the CPU oracle
(oracle/); everything else runs without a GPU.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def dev():
    from nn_b200.device import Device

    d = Device(0)
    yield d
    d.synchronize()


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle

    oracle.lib()
    return oracle
