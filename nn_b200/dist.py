"""One process per GPU: rendezvous for the library's NCCL communicator.

The reference is single-process and single-device; this is the launcher-side glue for the tensor-parallel decoder.
Rank 0 makes the NCCL id with ``ns_comm_unique_id``; the 128 bytes travel to the other ranks through a
``torch.distributed`` process group on the ``gloo`` backend (CPU sockets: no device memory, no collectives on the data
path), and every rank then calls ``ns_comm_init_rank`` on its own device.  RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR and
MASTER_PORT come from the launcher (``python -m torch.distributed.run``).
"""
from __future__ import annotations

import ctypes as C
import os

from . import native as N
from .device import Device


def env_rank() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def broadcast_bytes(payload: bytes | None, size: int, src: int = 0) -> bytes:
    """Sends `size` bytes from rank `src` to every rank over gloo (initialises the default group if needed)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        dist.init_process_group("gloo")
    buf = torch.zeros(size, dtype=torch.uint8)
    if dist.get_rank() == src:
        buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8).clone()
    dist.broadcast(buf, src)
    return bytes(buf.numpy().tobytes())


def init_comm(dev: Device):
    """Returns (comm handle or None, rank, world size)."""
    rank, world, _ = env_rank()
    if world == 1:
        return None, 0, 1
    # torch must load its own NCCL before the library opens "libnccl.so.2": the dynamic loader keeps one library per
    # soname, and torch's CUDA library needs symbols of the NCCL it was built with.
    import torch  # noqa: F401
    import torch.distributed  # noqa: F401
    ident = C.create_string_buffer(128)
    if rank == 0:
        N.call("ns_comm_unique_id", ident)
    data = broadcast_bytes(ident.raw if rank == 0 else None, 128)
    comm = C.c_void_p()
    N.call("ns_comm_init_rank", dev.handle, data, rank, world, C.byref(comm))
    return comm, rank, world


def make_peer_group(dev: Device, rank: int, world: int, slot_bytes: int):
    """A peer-memory group for ns_tp_reduce_norm_quant: every rank's 64-byte IPC handle is gathered over gloo."""
    import torch
    import torch.distributed as dist

    group = C.c_void_p()
    N.call("ns_peer_group_create", dev.handle, rank, world, C.c_uint64(slot_bytes), C.byref(group))
    mine = C.create_string_buffer(64)
    N.call("ns_peer_group_handle", group, mine)
    if world > 1:
        if not dist.is_initialized():
            dist.init_process_group("gloo")
        parts = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, torch.frombuffer(bytearray(mine.raw), dtype=torch.uint8).clone())
        handles = b"".join(bytes(t.numpy().tobytes()) for t in parts)
    else:
        handles = mine.raw
    N.call("ns_peer_group_connect", group, handles)
    return group


def barrier() -> None:
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()


def all_reduce_max(value: float) -> float:
    """Maximum of a host float over ranks (timing: the slowest rank counts)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        return value
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
