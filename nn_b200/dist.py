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


def all_gather_bytes(payload: bytes) -> list[bytes]:
    """Every rank's `payload` (same length everywhere), in rank order, over gloo."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        dist.init_process_group("gloo")
    parts = [torch.zeros(len(payload), dtype=torch.uint8) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, torch.frombuffer(bytearray(payload), dtype=torch.uint8).clone())
    return [bytes(t.numpy().tobytes()) for t in parts]


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


class PeerWatch:
    """Host-side failure detection for a multi-rank decoder, checked BETWEEN steps (no kernel or collective in flight).

    Every rank publishes the number of the step it is about to queue in a key-value store all ranks reach (the store of
    the torch.distributed rendezvous by default); before queuing step s a rank waits, for at most `timeout_s`, until
    every peer has published s.  A peer that left (crashed, or returned from its loop) never does: the waiting rank then
    tears its communicator down with `comm_abort` (ns_comm_abort: it must not wait for the missing peer) and raises
    NsError with NS_ERR_COMM, before anything that would wait for that peer on the GPU is launched.  `comm_error`, when
    given, is polled as well (ns_comm_async_error's result: non-zero = the transport itself reported a failure).
    The reference is single-process; the error convention is its CudaDriver.Check (Backends/Cuda/CudaDriver.cs:63-77).
    """

    NS_ERR_COMM = 5

    def __init__(self, rank: int, world: int, timeout_s: float = 30.0, store=None, comm_error=None, comm_abort=None, prefix: str = "ns_watch"):
        if store is None:
            import torch.distributed as dist
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s
        self.comm_error, self.comm_abort, self.prefix = comm_error, comm_abort, prefix
        self.aborted = False

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _fail(self, text: str):
        if self.comm_abort is not None and not self.aborted:
            self.comm_abort()
        self.aborted = True
        raise N.NsError("PeerWatch.check", self.NS_ERR_COMM, text)

    def check(self, step: int) -> None:
        """Call before queuing step `step` (0, 1, 2, ... in order)."""
        import time
        self.store.set(self._key(self.rank), str(step))
        deadline = time.monotonic() + self.timeout_s
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                if self.comm_error is not None:
                    code = self.comm_error()
                    if code:
                        self._fail(f"the transport reports error {code} before step {step}")
                seen = -1
                try:
                    if self.store.check([self._key(peer)]):
                        seen = int(self.store.get(self._key(peer)))
                except Exception as e:          # the store itself went away with the rank that served it
                    self._fail(f"rendezvous store unreachable before step {step}: {e}")
                if seen >= step:
                    break
                if time.monotonic() > deadline:
                    self._fail(f"rank {peer} did not reach step {step} within {self.timeout_s:.1f} s (last seen at step {seen})")
                time.sleep(0.005)
