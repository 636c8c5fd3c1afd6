"""nn_b200 -- sm_100a implementation of NeuralSharp's CUDA inference hot path behind its operator surface.

The package is a thin host layer over ``libns_b200.so`` (built from ``nn_b200/csrc``): ``native`` is the
ctypes binding, ``device`` the device/storage objects, ``backend`` the mirror of the reference's
``Backend`` operator surface, ``gpt`` the decoder driver.  Nothing here computes on the CPU.
"""
from . import native  # noqa: F401

__all__ = ["native"]
