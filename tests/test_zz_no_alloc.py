"""ns_qmatmul_i8_static -- the int8 product whose split-K partial sums live in a fixed array inside the library, for
hosts that cannot let the library allocate device memory (a decode step recorded into a CUDA graph without a warm-up
run; a host that accounts for every device block itself).  Checked against the regular entry point, bit for bit, on
two calls in a row that share the array, plus the size limit.  Collected last on purpose: if it fails under
`pytest -x`, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


def _operands(dev, orc, M, Nn, K, seed):
    aq, a_s = orc.quantize_rows_i8(orc.normal((M, K), seed))
    wq, w_s = orc.quantize_rows_i8(orc.normal((Nn, K), seed + 1, 0.02))
    bias = orc.normal((Nn,), seed + 2, 0.01)
    return [dev.from_numpy(x) for x in (aq, a_s, wq, w_s, bias)]


def _both(dev, ops, M, Nn, K, epilogue, out_dtype):
    a, a_s, w, w_s, b = ops
    y_ref, y_new = dev.empty(M * Nn, out_dtype), dev.empty(M * Nn, out_dtype)
    N.call("ns_qmatmul_i8", dev.handle, a.ptr, a_s.ptr, w.ptr, w_s.ptr, b.ptr, 0, 0, M, Nn, K, epilogue, out_dtype, y_ref.ptr, 0)
    N.call("ns_qmatmul_i8_static", dev.handle, a.ptr, a_s.ptr, w.ptr, w_s.ptr, b.ptr, 0, 0, M, Nn, K, epilogue, out_dtype, y_new.ptr)
    dev.synchronize()
    return y_ref.download(), y_new.download()


def test_matches_the_allocating_entry_point_twice_in_a_row(dev, orc):
    # decode shapes: K is split 4 ways (2 MiB of partial sums), then a different shape and epilogue reusing the array
    M, Nn, K = 64, 2048, 8192
    ref, new = _both(dev, _operands(dev, orc, M, Nn, K, 501), M, Nn, K, N.EPI_BIAS, N.NS_F32)
    assert np.array_equal(ref.view(np.uint32), new.view(np.uint32))        # tolerance 0: same kernels, same order
    # and directly against the oracle (same operands, regenerated on the host)
    aq, a_s = orc.quantize_rows_i8(orc.normal((M, K), 501))
    wq, w_s = orc.quantize_rows_i8(orc.normal((Nn, K), 502, 0.02))
    exp = orc.dequant_epilogue(orc.qmatmul_i8_acc(aq, wq), a_s, w_s, orc.normal((Nn,), 503, 0.01))
    assert np.array_equal(new.reshape(M, Nn).view(np.uint32), exp.view(np.uint32))
    M2, N2, K2 = 48, 1024, 4096
    ref, new = _both(dev, _operands(dev, orc, M2, N2, K2, 601), M2, N2, K2, N.EPI_BIAS_GELU, N.NS_BF16)
    assert np.array_equal(ref, new)
    # and the first shape again: stale partial sums of the second call must not leak into it
    ref, new = _both(dev, _operands(dev, orc, M, Nn, K, 701), M, Nn, K, N.EPI_NONE, N.NS_F32)
    assert np.array_equal(ref.view(np.uint32), new.view(np.uint32))


def test_rejects_shapes_beyond_the_fixed_array(dev, orc):
    M, Nn, K = 128, 4096, 4096
    ops = _operands(dev, orc, M, Nn, K, 801)
    y = dev.empty(M * Nn)
    dev.tune(64, 8)    # force an 8-way split: 8 * 128 * 4096 * 4 bytes = 16 MiB > 8 MiB
    try:
        with pytest.raises(N.NsError) as err:
            N.call("ns_qmatmul_i8_static", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, 0, 0, M, Nn, K, N.EPI_BIAS,
                   N.NS_F32, y.ptr)
        assert err.value.code == 3 and "fixed scratch array" in err.value.text
    finally:
        dev.tune(0, 0)
    dev.synchronize()


@pytest.mark.parametrize("M,Nn,K", [(4, 1024, 2048), (512, 1024, 1024)])
def test_shapes_that_need_no_partial_sums(dev, orc, M, Nn, K):
    """Four rows take the row-streaming kernel, 512 rows are not split along K: neither touches the fixed array, both must
    equal the regular entry point bit for bit."""
    ref, new = _both(dev, _operands(dev, orc, M, Nn, K, 901), M, Nn, K, N.EPI_BIAS, N.NS_F32)
    assert np.array_equal(ref.view(np.uint32), new.view(np.uint32))


def test_allocates_nothing_and_can_be_recorded(dev, orc):
    """The reason the entry point exists: free device memory is the same before and after calls with shapes it has not
    seen (the regular entry point would grow its scratch block), and after one warm call a call can be recorded into
    a graph and replayed."""
    import ctypes as C
    M, Nn, K = 32, 4096, 4096
    ops = _operands(dev, orc, 48, Nn, K, 951)      # 48 rows of activations; the calls below use the first m of them
    y = dev.empty(48 * Nn)
    y_ref = dev.empty(M * Nn)
    # one warm call with the kernels the shapes below use (the CUDA runtime loads a kernel's code on its first launch)
    N.call("ns_qmatmul_i8_static", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, 0, 0, 16, Nn, K, N.EPI_BIAS, N.NS_F32, y.ptr)
    dev.synchronize()

    def free_bytes():
        fr = C.c_uint64()
        N.call("ns_device_info", dev.handle, None, None, None, C.byref(fr))
        return fr.value

    before = free_bytes()
    for m in (24, 32, 48):       # shapes not seen before, all split along K
        N.call("ns_qmatmul_i8_static", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, 0, 0, m, Nn, K, N.EPI_BIAS, N.NS_F32, y.ptr)
    dev.synchronize()
    assert free_bytes() == before
    dev.capture_begin()
    try:
        N.call("ns_qmatmul_i8_static", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, 0, 0, M, Nn, K, N.EPI_BIAS, N.NS_F32, y.ptr)
    except Exception:
        N.call("ns_capture_abort", dev.handle)
        raise
    graph = dev.capture_end()
    N.call("ns_memset32_async", dev.handle, C.c_uint64(y.ptr), 0, C.c_uint64(M * Nn))
    dev.graph_launch(graph)
    N.call("ns_qmatmul_i8", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, 0, 0, M, Nn, K, N.EPI_BIAS, N.NS_F32, y_ref.ptr, 0)
    dev.synchronize()
    dev.graph_destroy(graph)
    assert np.array_equal(y.download(count=M * Nn).view(np.uint32), y_ref.download().view(np.uint32))


def test_rejects_an_unknown_residual_dtype(dev, orc):
    M, Nn, K = 16, 256, 512
    ops = _operands(dev, orc, M, Nn, K, 971)
    y = dev.empty(M * Nn)
    with pytest.raises(N.NsError) as err:
        N.call("ns_qmatmul_i8_static", dev.handle, ops[0].ptr, ops[1].ptr, ops[2].ptr, ops[3].ptr, ops[4].ptr, y.ptr, 7, M, Nn, K,
               N.EPI_BIAS_RESIDUAL, N.NS_F32, y.ptr)
    assert err.value.code == 2
