"""float32 operator surface (ns_f32_*) against the oracle, restating the reference's own tests:
MatMulReference / LargeTensors (tests/NeuralSharp.Tests/Program.cs:329-368,406-418), BatchedMatMul
(AdvancedTests.cs:195-233), SoftmaxReference / ArgMaxAndAccuracy (AdvancedTests.cs:162-193), FusedKernels
(DecodingTests.cs:34-67).  Products are compared bit-exactly (same fused-multiply-add chain), the row-wise
operators within the reference's tolerances.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


def _mm(dev, a, b, c0, batch, m, n, k, ta, tb, beta):
    d_a, d_b = dev.from_numpy(a), dev.from_numpy(b)
    d_c = dev.from_numpy(c0)
    N.call("ns_f32_batched_matmul", dev.handle, d_a.ptr, d_b.ptr, d_c.ptr, batch, m, n, k, int(ta), int(tb), C.c_float(beta))
    dev.synchronize()
    return d_c.download((batch, m, n))


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 2), (17, 33, 9), (64, 48, 70), (130, 67, 91)])
def test_matmul_reference(dev, orc, m, n, k):
    for ta in (False, True):
        for tb in (False, True):
            for beta in (0.0, 1.0):
                a = orc.normal((k, m) if ta else (m, k), 1 + m)
                b = orc.normal((n, k) if tb else (k, n), 2 + n)
                c0 = orc.normal((1, m, n), 3 + k)
                got = _mm(dev, a, b, c0, 1, m, n, k, ta, tb, beta)
                exp = orc.matmul_f32(a, b, 1, m, n, k, ta, tb, beta, c=c0)
                assert np.array_equal(got.view(np.uint32), exp.view(np.uint32)), (m, n, k, ta, tb, beta, orc.max_err(exp, got))
                # and against double accumulation, the reference test's own check (tolerance 1e-4)
                A = (a.T if ta else a).astype(np.float64)
                B = (b.T if tb else b).astype(np.float64)
                assert orc.close(A @ B + beta * c0[0], got[0], 1e-4)


def test_large_tensors(dev, orc):
    a = orc.normal((1000, 1000), 9)
    ones = np.ones((1000, 1), np.float32)
    got = _mm(dev, a, ones, np.zeros((1, 1000, 1), np.float32), 1, 1000, 1, 1000, False, False, 0.0)
    assert orc.close(a.astype(np.float64).sum(axis=1), got[0, :, 0], 1e-3)


def test_batched_matmul(dev, orc):
    for ta in (False, True):
        for tb in (False, True):
            a = orc.normal((3, 4, 5) if ta else (3, 5, 4), 31)
            b = orc.normal((3, 6, 4) if tb else (3, 4, 6), 32)
            got = _mm(dev, a, b, np.zeros((3, 5, 6), np.float32), 3, 5, 6, 4, ta, tb, 0.0)
            exp = orc.matmul_f32(a, b, 3, 5, 6, 4, ta, tb)
            assert np.array_equal(got, exp)


def test_softmax_kat_and_fused(dev, orc):
    x = dev.from_numpy(np.array([1000.0, 0.0, -1000.0], np.float32))
    y = dev.empty(3)
    N.call("ns_f32_scale_mask_softmax", dev.handle, x.ptr, 0, y.ptr, 1, 3, 1, C.c_float(1.0))
    dev.synchronize()
    assert orc.close([1.0, 0.0, 0.0], y.download(), 1e-6)
    # FusedKernels: scale + mask + softmax == (x * 0.7 + mask).Softmax(), tolerance 1e-5
    rows, cols = 6, 37
    xs = orc.normal((rows, cols), 41, 3.0)
    mask = np.where(np.arange(cols)[None, :] <= np.arange(3)[:, None] + 20, 0.0, -1e9).astype(np.float32)
    dx, dm, dy = dev.from_numpy(xs), dev.from_numpy(mask), dev.empty(rows * cols)
    N.call("ns_f32_scale_mask_softmax", dev.handle, dx.ptr, dm.ptr, dy.ptr, rows, cols, 3, C.c_float(0.7))
    dev.synchronize()
    got = dy.download((rows, cols))
    assert orc.close(orc.scale_mask_softmax(xs, mask, 0.7), got, 1e-5)
    unfused = orc.softmax(xs * np.float32(0.7) + np.tile(mask, (2, 1)))
    assert orc.close(unfused, got, 1e-5)
    assert orc.close(np.ones(rows), got.sum(axis=1), 1e-5)


def test_layernorm_and_bias_gelu(dev, orc):
    rows, cols = 9, 200
    x = orc.normal((rows, cols), 51, 2.0)
    g, b = orc.normal((cols,), 52), orc.normal((cols,), 53)
    dx, dg, db, dy = dev.from_numpy(x), dev.from_numpy(g), dev.from_numpy(b), dev.empty(rows * cols)
    N.call("ns_f32_layernorm_fused", dev.handle, dx.ptr, dg.ptr, db.ptr, dy.ptr, rows, cols, C.c_float(1e-5))
    N.call("ns_f32_bias_gelu", dev.handle, dx.ptr, dg.ptr, dx.ptr, C.c_int64(rows * cols), cols)
    dev.synchronize()
    assert orc.close(orc.layernorm_fused(x, g, b), dy.download((rows, cols)), 1e-4)
    assert orc.close(orc.bias_gelu(x, g), dx.download((rows, cols)), 1e-5)


def test_argmax_kat(dev, orc):
    p = np.array([[0.1, 0.7, 0.2], [0.5, 0.2, 0.3], [0.2, 0.2, 0.6], [0.3, 0.4, 0.3]], np.float32)
    dp, dy = dev.from_numpy(p), dev.empty(4)
    N.call("ns_f32_argmax", dev.handle, dp.ptr, dy.ptr, 4, 3)
    dev.synchronize()
    assert list(dy.download()) == [1.0, 0.0, 2.0, 1.0]
    # ties: first maximum wins, also across threads and warps
    x = np.zeros((3, 5000), np.float32)
    x[0, [4999, 300, 77]] = 5.0
    x[1, :] = -1.0
    x[2, 4097] = 1.0
    dx, dy = dev.from_numpy(x), dev.empty(3)
    N.call("ns_f32_argmax", dev.handle, dx.ptr, dy.ptr, 3, 5000)
    dev.synchronize()
    assert list(dy.download()) == [77.0, 0.0, 4097.0]
    assert np.array_equal(orc.argmax(x), dy.download())


def test_decoding_primitives(dev, orc):
    heads, steps, cap, dim = 6, 3, 12, 8
    pos = np.array([4.0], np.float32)
    src = orc.normal((heads, steps, dim), 61)
    cache = np.zeros((heads, cap, dim), np.float32)
    dpos, dsrc, dcache = dev.from_numpy(pos), dev.from_numpy(src), dev.from_numpy(cache)
    dmask = dev.empty(steps * cap)
    N.call("ns_f32_key_value_write", dev.handle, dsrc.ptr, dcache.ptr, dpos.ptr, heads, steps, cap, dim)
    N.call("ns_f32_decoder_mask", dev.handle, dpos.ptr, dmask.ptr, steps, cap)
    N.call("ns_f32_affine", dev.handle, dpos.ptr, dpos.ptr, C.c_int64(1), C.c_float(1.0), C.c_float(steps))
    dev.synchronize()
    orc.kv_write(src, cache, 4.0)
    assert np.array_equal(cache, dcache.download((heads, cap, dim)))
    assert np.array_equal(orc.decoder_mask(4.0, steps, cap), dmask.download((steps, cap)))
    assert dpos.download()[0] == 7.0
    # gather + add row vector + add
    table = orc.normal((11, 16), 62)
    ids = np.array([3, 0, 10, 10, 7], np.float32)
    dt, di, dy = dev.from_numpy(table), dev.from_numpy(ids), dev.empty(5 * 16)
    N.call("ns_f32_gather", dev.handle, dt.ptr, di.ptr, dy.ptr, 5, 16, 11)
    v = orc.normal((16,), 63)
    dv = dev.from_numpy(v)
    N.call("ns_f32_add_row_vector", dev.handle, dy.ptr, dv.ptr, dy.ptr, 5, 16)
    dev.synchronize()
    assert np.array_equal(orc.add_rowvec(orc.gather(table, ids), v), dy.download((5, 16)))


def test_permute_and_copy2d(dev, orc):
    # head split as MultiHeadAttention does it: narrow on the last dim (copy2d), [n,t,H,dh] -> [n,H,t,dh] (permute)
    n, t, H, dh = 2, 3, 4, 5
    D = H * dh
    qkv = orc.normal((n * t, 3 * D), 71)
    dq, dpart, dperm = dev.from_numpy(qkv), dev.empty(n * t * D), dev.empty(n * t * D)
    N.call("ns_f32_copy2d", dev.handle, dq.ptr, C.c_int64(D), 3 * D, dpart.ptr, C.c_int64(0), D, n * t, D, 0)
    shape = (C.c_int * 4)(n, H, t, dh)
    strides = (C.c_int * 4)(t * D, dh, D, 1)
    N.call("ns_f32_permute", dev.handle, dpart.ptr, dperm.ptr, shape, strides, 4, 0)
    dev.synchronize()
    exp = qkv[:, D:2 * D].reshape(n, t, H, dh).transpose(0, 2, 1, 3)
    assert np.array_equal(exp, dperm.download((n, H, t, dh)))
