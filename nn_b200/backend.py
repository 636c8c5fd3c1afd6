"""The reference's operator surface, method for method, over the C ABI.

``NsB200Backend`` is the Python twin of the C# class a maintainer would write as ``NsB200Backend : Backend``
(src/NeuralSharp/Backends/Backend.cs:66-282): same method names, same argument lists, ``Storage`` handles in place
of the reference's ``Storage``.  Only the methods one cached decoder step calls are present; everything else of
``Backend`` (training, convolution, optimisers) is outside this library.  All storage here is float32, as in
the reference ("contiguous row-major float32 buffers", Backend.cs:60-65).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import native as N
from .device import Device, Storage


class NsB200Backend:
    def __init__(self, device: Device):
        self.device = device
        self._h = device.handle

    # ---- memory (Backend.cs:68-86)
    def Allocate(self, length: int, zeroed: bool = False) -> Storage:
        return Storage(self.device, length, N.NS_F32, zeroed)

    def Return(self, storage: Storage) -> None:
        storage.release()

    def Upload(self, source, destination: Storage) -> None:
        destination.upload(np.asarray(source, dtype=np.float32))

    def Download(self, source: Storage) -> np.ndarray:
        return source.download()

    def DownloadRange(self, source: Storage, offset: int, count: int) -> np.ndarray:
        return source.download(offset=offset, count=count)

    def Fill(self, y: Storage, n: int, value: float) -> None:
        bits = int(np.float32(value).view(np.uint32))
        N.call("ns_memset32_async", self._h, C.c_uint64(y.ptr), bits, C.c_uint64(n))

    def Copy(self, x: Storage, y: Storage, n: int) -> None:
        N.call("ns_d2d_async", self._h, C.c_uint64(y.ptr), C.c_uint64(x.ptr), C.c_uint64(4 * n))

    def Synchronize(self) -> None:
        self.device.synchronize()

    # ---- element-wise (Backend.cs:95-119)
    def Add(self, a: Storage, b: Storage, c: Storage, n: int) -> None:
        """Binary(BinaryOp.Add, a, b, c, n)."""
        N.call("ns_f32_add", self._h, a.ptr, b.ptr, c.ptr, C.c_int64(n))

    def Affine(self, x: Storage, y: Storage, n: int, alpha: float, beta: float) -> None:
        N.call("ns_f32_affine", self._h, x.ptr, y.ptr, C.c_int64(n), C.c_float(alpha), C.c_float(beta))

    def AddRowVector(self, a: Storage, v: Storage, c: Storage, rows: int, cols: int) -> None:
        N.call("ns_f32_add_row_vector", self._h, a.ptr, v.ptr, c.ptr, rows, cols)

    def AddBroadcastScalar(self, s: Storage, y: Storage, n: int, scale: float) -> None:
        N.call("ns_f32_add_broadcast_scalar", self._h, s.ptr, y.ptr, C.c_int64(n), C.c_float(scale))

    # ---- products (Backend.cs:121-129)
    def BatchedMatMul(self, a: Storage, b: Storage, c: Storage, batch: int, m: int, n: int, k: int, transA: bool, transB: bool, beta: float,
                      a_offset: int = 0, b_offset: int = 0, c_offset: int = 0) -> None:
        N.call("ns_f32_batched_matmul", self._h, C.c_uint64(a.ptr + 4 * a_offset), C.c_uint64(b.ptr + 4 * b_offset), C.c_uint64(c.ptr + 4 * c_offset),
               batch, m, n, k, int(transA), int(transB), C.c_float(beta))

    def MatMul(self, a, b, c, m, n, k, transA, transB, beta) -> None:
        self.BatchedMatMul(a, b, c, 1, m, n, k, transA, transB, beta)

    # ---- shape operators (Backend.cs:140,172,193,199)
    def ArgMax(self, x: Storage, y: Storage, rows: int, cols: int) -> None:
        N.call("ns_f32_argmax", self._h, x.ptr, y.ptr, rows, cols)

    def ArgMaxRows(self, x: Storage, y: Storage, rows: int, cols: int, rowStride: int, rowOffset: int) -> None:
        """Greedy choice with the sampler's row addressing (row r at r * rowStride + rowOffset, Backend.cs:248)."""
        N.call("ns_f32_argmax_strided", self._h, x.ptr, y.ptr, rows, cols, C.c_int64(rowStride), C.c_int64(rowOffset))

    def Gather(self, table: Storage, indices: Storage, y: Storage, count: int, dim: int, vocabulary: int) -> None:
        N.call("ns_f32_gather", self._h, table.ptr, indices.ptr, y.ptr, count, dim, vocabulary)

    def Permute(self, x: Storage, y: Storage, outShape, inStrides, accumulate: bool = False) -> None:
        r = len(outShape)
        N.call("ns_f32_permute", self._h, x.ptr, y.ptr, (C.c_int * r)(*outShape), (C.c_int * r)(*inStrides), r, int(accumulate))

    def Copy2D(self, src: Storage, srcOffset: int, srcStride: int, dst: Storage, dstOffset: int, dstStride: int, rows: int, cols: int,
               accumulate: bool = False) -> None:
        N.call("ns_f32_copy2d", self._h, src.ptr, C.c_int64(srcOffset), srcStride, dst.ptr, C.c_int64(dstOffset), dstStride, rows, cols, int(accumulate))

    # ---- fused inference kernels (Backend.cs:221-230)
    def ScaleMaskSoftmax(self, x: Storage, mask, y: Storage, rows: int, cols: int, maskRows: int, scale: float) -> None:
        N.call("ns_f32_scale_mask_softmax", self._h, x.ptr, mask.ptr if mask is not None else 0, y.ptr, rows, cols, maskRows, C.c_float(scale))

    def LayerNormFused(self, x: Storage, gamma: Storage, beta: Storage, y: Storage, rows: int, cols: int, eps: float) -> None:
        N.call("ns_f32_layernorm_fused", self._h, x.ptr, gamma.ptr, beta.ptr, y.ptr, rows, cols, C.c_float(eps))

    def BiasGelu(self, x: Storage, bias: Storage, y: Storage, n: int, cols: int) -> None:
        N.call("ns_f32_bias_gelu", self._h, x.ptr, bias.ptr, y.ptr, C.c_int64(n), cols)

    # ---- incremental decoding (Backend.cs:232-238)
    def DecoderMask(self, position: Storage, mask: Storage, rows: int, capacity: int) -> None:
        N.call("ns_f32_decoder_mask", self._h, position.ptr, mask.ptr, rows, capacity)

    def KeyValueWrite(self, source: Storage, cache: Storage, position: Storage, heads: int, steps: int, capacity: int, dim: int) -> None:
        N.call("ns_f32_key_value_write", self._h, source.ptr, cache.ptr, position.ptr, heads, steps, capacity, dim)

    # ---- on-device sampling (Backend.cs:240-261)
    def SampleRows(self, logits: Storage, ids: Storage, stats: Storage, step: Storage, rows: int, vocabulary: int, rowStride: int, rowOffset: int,
                   temperature: float, topK: int, topP: float, minP: float, seed: int) -> None:
        N.call("ns_f32_sample_rows", self._h, logits.ptr, ids.ptr, stats.ptr, step.ptr, rows, vocabulary, rowStride, rowOffset,
               C.c_float(temperature), topK, C.c_float(topP), C.c_float(minP), C.c_uint32(seed & 0xFFFFFFFF))

    def PenalizeRows(self, logits: Storage, work: Storage, history: Storage, length: Storage, rows: int, vocabulary: int, rowStride: int,
                     rowOffset: int, capacity: int, lastN: int, repeat: float, presence: float, frequency: float) -> None:
        N.call("ns_f32_penalize_rows", self._h, logits.ptr, work.ptr, history.ptr, length.ptr, rows, vocabulary, rowStride, rowOffset,
               capacity, lastN, C.c_float(repeat), C.c_float(presence), C.c_float(frequency))

    def HistoryPush(self, ids: Storage, history: Storage, length: Storage, rows: int, capacity: int) -> None:
        N.call("ns_f32_history_push", self._h, ids.ptr, history.ptr, length.ptr, rows, capacity)

    # ---- graphs (Backend.cs:266-281)
    SupportsGraphs = True

    def BeginCapture(self) -> None:
        self.device.capture_begin()

    def EndCapture(self):
        return self.device.capture_end()

    def AbortCapture(self) -> None:
        N.call("ns_capture_abort", self._h)

    def ReplayGraph(self, graph) -> None:
        self.device.graph_launch(graph)

    def DestroyGraph(self, graph) -> None:
        self.device.graph_destroy(graph)
