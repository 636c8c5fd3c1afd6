"""ns_linear_forward_host: float32 host rows in, float32 host rows out, chunks pipelined over three streams.

Row-wise quantisation and the product are independent per row, so the chunked result must equal the oracle's
unchunked W8A8 Linear bit for bit whatever the chunk size (ragged last chunk, one chunk, more chunks than buffer
slots), for pinned and pageable host memory, and when called back to back.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


def _linear(dev, w_kn, bias, mode=N.NS_I8):
    h = C.c_void_p()
    w = np.ascontiguousarray(w_kn, np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    N.call("ns_linear_create", dev.handle, w.shape[0], w.shape[1], mode, w.ctypes.data_as(C.POINTER(C.c_float)),
           None if b is None else b.ctypes.data_as(C.POINTER(C.c_float)), N.SPLIT_NONE, 1, 0, 1, C.byref(h))
    return h


def _oracle(orc, x, w_kn, bias, act):
    xq, xs = orc.quantize_rows_i8(x)
    wq, ws = orc.quantize_rows_i8(np.ascontiguousarray(w_kn.T))
    return orc.dequant_epilogue(orc.qmatmul_i8_acc(xq, wq), xs, ws, bias=bias, act=act)


@pytest.mark.parametrize("M,K,NN,chunk", [(1, 64, 48, 0), (300, 256, 192, 128), (1000, 128, 320, 96), (517, 512, 64, 517), (2048, 1024, 1024, 0)])
@pytest.mark.parametrize("epi", [N.EPI_NONE, N.EPI_BIAS, N.EPI_BIAS_GELU])
def test_host_forward_equals_oracle(dev, orc, M, K, NN, chunk, epi):
    x = orc.normal((M, K), 10 + M)
    w = orc.normal((K, NN), 11 + K, 0.05)
    bias = orc.normal((NN,), 12, 0.1)
    lin = _linear(dev, w, bias)
    y = np.full((M, NN), np.nan, np.float32)
    N.call("ns_linear_forward_host", dev.handle, lin, x.ctypes.data_as(C.c_void_p), M, epi, y.ctypes.data_as(C.c_void_p), chunk)
    dev.synchronize()
    exp = _oracle(orc, x, w, bias if epi != N.EPI_NONE else None, 1 if epi == N.EPI_BIAS_GELU else 0)
    if epi == N.EPI_BIAS_GELU:
        assert orc.close(exp, y, 1e-6)          # tanhf of the device and of the host's libm differ in the last place
    else:
        assert np.array_equal(y.view(np.uint32), exp.view(np.uint32)), orc.max_err(exp, y)
    N.call("ns_linear_destroy", lin)


def test_pinned_back_to_back_and_growth(dev, orc):
    """Two different inputs through the same staging slots with nothing but stream order between the calls; then a
    larger chunk (the staging buffers grow) and a smaller one."""
    M, K, NN = 1536, 512, 768
    w = orc.normal((K, NN), 3, 0.05)
    bias = orc.normal((NN,), 4, 0.1)
    lin = _linear(dev, w, bias)
    hx, hy = C.c_void_p(), C.c_void_p()
    N.call("ns_host_alloc", C.c_uint64(2 * M * K * 4), C.byref(hx))
    N.call("ns_host_alloc", C.c_uint64(2 * M * NN * 4), C.byref(hy))
    X = np.ctypeslib.as_array(C.cast(hx, C.POINTER(C.c_float)), (2, M, K))
    Y = np.ctypeslib.as_array(C.cast(hy, C.POINTER(C.c_float)), (2, M, NN))
    X[0], X[1] = orc.normal((M, K), 5), orc.normal((M, K), 6)
    for chunk in (128, 1024, 256):
        Y[:] = np.nan
        for i in range(2):
            N.call("ns_linear_forward_host", dev.handle, lin, C.c_void_p(hx.value + i * M * K * 4), M, N.EPI_BIAS,
                   C.c_void_p(hy.value + i * M * NN * 4), chunk)
        dev.synchronize()
        for i in range(2):
            exp = _oracle(orc, X[i], w, bias, 0)
            assert np.array_equal(Y[i].view(np.uint32), exp.view(np.uint32)), (chunk, i)
    N.call("ns_linear_destroy", lin)
    N.call("ns_host_free", hx)
    N.call("ns_host_free", hy)


def test_bf16_layer_and_errors(dev, orc):
    M, K, NN = 200, 128, 96
    x, w = orc.normal((M, K), 1), orc.normal((K, NN), 2, 0.05)
    lin = _linear(dev, w, None, mode=N.NS_BF16)
    y = np.zeros((M, NN), np.float32)
    N.call("ns_linear_forward_host", dev.handle, lin, x.ctypes.data_as(C.c_void_p), M, N.EPI_NONE, y.ctypes.data_as(C.c_void_p), 64)
    dev.synchronize()
    exp = orc.matmul_bf16(orc.round_bf16(x), orc.round_bf16(np.ascontiguousarray(w.T)), True)
    assert orc.close(exp, y, 1e-4)
    with pytest.raises(N.NsError, match="no bias"):
        N.call("ns_linear_forward_host", dev.handle, lin, x.ctypes.data_as(C.c_void_p), M, N.EPI_BIAS, y.ctypes.data_as(C.c_void_p), 64)
    with pytest.raises(N.NsError, match="epilogue must be"):
        N.call("ns_linear_forward_host", dev.handle, lin, x.ctypes.data_as(C.c_void_p), M, N.EPI_BIAS_RESIDUAL, y.ctypes.data_as(C.c_void_p), 64)
    with pytest.raises(N.NsError, match="null argument"):
        N.call("ns_linear_forward_host", dev.handle, lin, None, M, N.EPI_NONE, y.ctypes.data_as(C.c_void_p), 64)
    dev.capture_begin()
    try:
        with pytest.raises(N.NsError, match="cannot be captured"):
            N.call("ns_linear_forward_host", dev.handle, lin, x.ctypes.data_as(C.c_void_p), M, N.EPI_NONE, y.ctypes.data_as(C.c_void_p), 64)
    finally:
        N.call("ns_capture_abort", dev.handle)
    N.call("ns_linear_destroy", lin)
