"""Device object and storage blocks over the C ABI.

``Device`` plays the part of the reference's ``CudaBackend`` instance (one per ordinal, one stream:
src/NeuralSharp/Backends/Cuda/CudaBackend.cs:17-100) and ``Storage`` the part of its ``Storage`` /
``CudaStorage`` (Backends/Backend.cs:41-58, CudaBackend.cs:7-10): a block of device memory with a
length, released explicitly or when collected.  numpy arrays are the host side of Upload / Download
(Backend.cs:77-82).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import native as N

_NP = {N.NS_F32: np.float32, N.NS_BF16: np.uint16, N.NS_I8: np.int8, N.NS_I32: np.int32}
_SIZE = {N.NS_F32: 4, N.NS_BF16: 2, N.NS_I8: 1, N.NS_I32: 4}


class Storage:
    """A block of device memory holding ``count`` elements of ``dtype`` (NS_F32 / NS_BF16 / NS_I8 / NS_I32)."""

    def __init__(self, device: "Device", count: int, dtype: int = N.NS_F32, zeroed: bool = False):
        self.device, self.count, self.dtype = device, int(count), dtype
        ptr = C.c_uint64(0)
        N.call("ns_alloc", device.handle, C.c_uint64(self.nbytes), int(zeroed), C.byref(ptr))
        self.ptr = ptr.value

    @property
    def nbytes(self) -> int:
        return self.count * _SIZE[self.dtype]

    def upload(self, host) -> "Storage":
        a = np.ascontiguousarray(host, dtype=_NP[self.dtype])
        if a.size != self.count:
            raise ValueError(f"upload of {a.size} elements into a storage of {self.count}")
        N.call("ns_h2d", self.device.handle, C.c_uint64(self.ptr), a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes))
        return self

    def download(self, shape=None, offset: int = 0, count: int | None = None) -> np.ndarray:
        count = self.count - offset if count is None else count
        out = np.empty(count, dtype=_NP[self.dtype])
        if count:
            N.call("ns_d2h", self.device.handle, out.ctypes.data_as(C.c_void_p),
                   C.c_uint64(self.ptr + offset * _SIZE[self.dtype]), C.c_uint64(out.nbytes))
        return out if shape is None else out.reshape(shape)

    def release(self) -> None:
        if self.ptr:
            N.call("ns_free", self.device.handle, C.c_uint64(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            if self.ptr and self.device.handle:
                N.load().ns_free(self.device.handle, C.c_uint64(self.ptr))
        except Exception:
            pass


class Device:
    """One B200 and its stream.  Every operator call is queued on that stream."""

    def __init__(self, ordinal: int = 0, stream: int | None = None):
        N.load()
        h = C.c_void_p()
        if stream is None:
            N.call("ns_device_open", ordinal, C.byref(h))
        else:
            N.call("ns_device_open_on_stream", ordinal, C.c_uint64(stream), C.byref(h))
        self.handle = h
        self.ordinal = ordinal
        name = C.create_string_buffer(128)
        sms, tot, free = C.c_int(), C.c_uint64(), C.c_uint64()
        N.call("ns_device_info", h, name, C.byref(sms), C.byref(tot), C.byref(free))
        self.name, self.sm_count, self.total_bytes = name.value.decode(), sms.value, tot.value

    @staticmethod
    def count() -> int:
        n = C.c_int()
        N.call("ns_device_count", C.byref(n))
        return n.value

    # ---- memory
    def empty(self, count: int, dtype: int = N.NS_F32) -> Storage:
        return Storage(self, count, dtype)

    def zeros(self, count: int, dtype: int = N.NS_F32) -> Storage:
        return Storage(self, count, dtype, zeroed=True)

    def from_numpy(self, a: np.ndarray, dtype: int | None = None) -> Storage:
        if dtype is None:
            dtype = {np.dtype(np.float32): N.NS_F32, np.dtype(np.uint16): N.NS_BF16, np.dtype(np.int8): N.NS_I8,
                     np.dtype(np.int32): N.NS_I32}[np.asarray(a).dtype]
        return Storage(self, np.asarray(a).size, dtype).upload(a)

    def synchronize(self) -> None:
        N.call("ns_stream_sync", self.handle)

    def stream(self) -> int:
        s = C.c_uint64()
        N.call("ns_device_stream", self.handle, C.byref(s))
        return s.value

    def tune(self, tile_n: int = 0, k_splits: int = 0) -> None:
        N.call("ns_device_tune", self.handle, tile_n, k_splits)

    def close(self) -> None:
        if self.handle:
            N.call("ns_device_close", self.handle)
            self.handle = None

    # ---- events
    def event(self) -> int:
        e = C.c_uint64()
        N.call("ns_event_create", self.handle, C.byref(e))
        return e.value

    def record(self, event: int) -> None:
        N.call("ns_event_record", self.handle, C.c_uint64(event))

    def wait_event(self, event: int) -> None:
        """Work queued on this device object's stream from now on waits for `event` (recorded on any stream of the GPU)."""
        N.call("ns_stream_wait_event", self.handle, C.c_uint64(event))

    def elapsed_ms(self, start: int, stop: int) -> float:
        ms = C.c_float()
        N.call("ns_event_elapsed_ms", self.handle, C.c_uint64(start), C.c_uint64(stop), C.byref(ms))
        return ms.value

    # ---- graphs (Backend.BeginCapture / EndCapture / ReplayGraph, Backends/Backend.cs:266-281)
    def capture_begin(self) -> None:
        N.call("ns_capture_begin", self.handle)

    def capture_end(self) -> C.c_void_p:
        g = C.c_void_p()
        N.call("ns_capture_end", self.handle, C.byref(g))
        return g

    def graph_launch(self, graph) -> None:
        N.call("ns_graph_launch", self.handle, graph)

    def graph_destroy(self, graph) -> None:
        N.call("ns_graph_destroy", graph)
