"""Row-wise operators of the bf16 / int8 path against the oracle: quantisation bit-exact, LayerNorm within
1e-4 (float output) / one bf16 ulp, fused LayerNorm -> int8 against the same composition in the oracle."""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 16), (5, 100), (64, 2048), (33, 8192), (130, 512), (2500, 2048), (2100, 4096), (2049, 1024),
                                       (2060, 8192), (20000, 2048), (10000, 8192), (9000, 4096), (30000, 1024)])
def test_quantize_rows_bit_exact(dev, orc, rows, cols):
    """The many-row cases are sized so that every row group of the streaming kernels goes round its ring of buffers more than once."""
    x = orc.normal((rows, cols), 81, 1.5)
    x[0, :] = 0.0  # all-zero row -> scale 1
    if rows > 2:
        x[2, 0] = 1e-30
    if rows > 3:
        # scale exactly 1 and quotients on half-integers: ties go to even, through the kernels' exact-division path
        x[3, :] = np.clip(x[3, :] * 20.0, -126.0, 126.0)
        x[3, :16] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, 126.5, -126.5, 63.5, 64.5, -3.5, 4.5, 0.25, 0.75, -0.75, 100.5]
    for dtype, host in ((N.NS_F32, x), (N.NS_BF16, orc.round_bf16(x))):
        dx = dev.from_numpy(host)
        dq, ds = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
        N.call("ns_quantize_rows_i8", dev.handle, dx.ptr, dtype, C.c_int64(rows), cols, dq.ptr, ds.ptr)
        dev.synchronize()
        q, s = orc.quantize_rows_i8(host)
        assert np.array_equal(s, ds.download())
        assert np.array_equal(q, dq.download((rows, cols)))


@pytest.mark.parametrize("cols", [1024, 2048, 8192])
def test_quantize_rows_odd_values_agree_between_kernels(dev, orc, cols):
    """Rows with NaNs, infinities or only subnormal values: the many-row kernels find them by their maximum and round them with
    the plain divisions, so they must give the bytes and scales the few-row kernel (a CTA per row) gives for the same rows."""
    rows = 2100
    x = orc.round_bf16(orc.normal((rows, cols), 83, 1.5)).copy()
    x[5, 7] = 0x7FC0                                  # NaN
    x[9, 100] = 0x7F80                                # +infinity
    x[11, 3], x[11, 900] = 0xFF80, 0x7FC0             # -infinity and a NaN
    x[20, :] = (np.arange(cols) % 0x7F + 1).astype(np.uint16)          # subnormals only: the scale has no float reciprocal
    x[21, :] = 0x8001
    x[30, :] = 0x7FC0                                 # nothing but NaNs
    dx = dev.from_numpy(x)
    dq, ds = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
    N.call("ns_quantize_rows_i8", dev.handle, dx.ptr, N.NS_BF16, C.c_int64(rows), cols, dq.ptr, ds.ptr)
    dq2, ds2 = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
    for r0 in range(0, rows, 700):
        N.call("ns_quantize_rows_i8", dev.handle, C.c_uint64(dx.ptr + r0 * cols * 2), N.NS_BF16, C.c_int64(700), cols, C.c_uint64(dq2.ptr + r0 * cols),
               C.c_uint64(ds2.ptr + r0 * 4))
    dev.synchronize()
    assert np.array_equal(ds.download().view(np.uint32), ds2.download().view(np.uint32))
    assert np.array_equal(dq.download((rows, cols)), dq2.download((rows, cols)))
    # and the untouched rows follow the rule
    q, sc = orc.quantize_rows_i8(x[100:200])
    assert np.array_equal(q, dq.download((rows, cols))[100:200]) and np.array_equal(sc, ds.download()[100:200])


@pytest.mark.parametrize("cols", [1024, 2048, 4096])
def test_layernorm_int8_is_the_same_in_both_kernel_families(dev, orc, cols):
    """2100 rows at once take the many-row kernel, the same rows 700 at a time the few-row kernel (a CTA per row).  Both sum a
    row vector by vector, 32 vectors by the same shuffle tree, piece after piece, so that a sequence read in a large batch and
    the same sequence read alone get the same bits."""
    rows = 2100
    x = orc.round_bf16(orc.normal((rows, cols), 95, 2.0))
    g, b = orc.normal((cols,), 96, 0.5, 1.0), orc.normal((cols,), 97, 0.1)
    dx, dg, db = dev.from_numpy(x), dev.from_numpy(g), dev.from_numpy(b)
    q1, s1 = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
    N.call("ns_layernorm", dev.handle, dx.ptr, N.NS_BF16, dg.ptr, db.ptr, C.c_int64(rows), cols, C.c_float(1e-5), N.NS_I8, q1.ptr, s1.ptr)
    q2, s2 = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
    for r0 in range(0, rows, 700):
        N.call("ns_layernorm", dev.handle, C.c_uint64(dx.ptr + r0 * cols * 2), N.NS_BF16, dg.ptr, db.ptr, C.c_int64(700), cols, C.c_float(1e-5), N.NS_I8,
               C.c_uint64(q2.ptr + r0 * cols), C.c_uint64(s2.ptr + r0 * 4))
    dev.synchronize()
    assert np.array_equal(s1.download().view(np.uint32), s2.download().view(np.uint32))
    assert np.array_equal(q1.download((rows, cols)), q2.download((rows, cols)))


@pytest.mark.parametrize("rows,cols", [(3, 128), (64, 2048), (7, 8192), (40, 512), (2500, 2048), (2049, 1024), (2050, 4096), (20000, 2048),
                                       (30000, 1024)])
def test_layernorm_variants(dev, orc, rows, cols):
    x = orc.normal((rows, cols), 91, 2.0)
    g, b = orc.normal((cols,), 92, 0.5, 1.0), orc.normal((cols,), 93, 0.1)
    exp = orc.layernorm_fused(x, g, b)
    dg, db = dev.from_numpy(g), dev.from_numpy(b)
    dx = dev.from_numpy(x)
    dy = dev.empty(rows * cols)
    N.call("ns_layernorm", dev.handle, dx.ptr, N.NS_F32, dg.ptr, db.ptr, C.c_int64(rows), cols, C.c_float(1e-5), N.NS_F32, dy.ptr, 0)
    dev.synchronize()
    assert orc.close(exp, dy.download((rows, cols)), 1e-4)
    # bf16 in, int8 out: compare with the oracle composition on the same bf16 input; the statistics are summed in a
    # different order, so a value on a rounding boundary may move by one step: allow |dq| <= 1 on < 0.1 % of elements
    xb = orc.round_bf16(x)
    expb = orc.layernorm_fused(orc.widen_bf16(xb), g, b)
    q_exp, s_exp = orc.quantize_rows_i8(orc.round_bf16(expb))
    dxb = dev.from_numpy(xb)
    dq, ds = dev.empty(rows * cols, N.NS_I8), dev.empty(rows)
    N.call("ns_layernorm", dev.handle, dxb.ptr, N.NS_BF16, dg.ptr, db.ptr, C.c_int64(rows), cols, C.c_float(1e-5), N.NS_I8, dq.ptr, ds.ptr)
    dyb = dev.empty(rows * cols, N.NS_BF16)
    N.call("ns_layernorm", dev.handle, dxb.ptr, N.NS_BF16, dg.ptr, db.ptr, C.c_int64(rows), cols, C.c_float(1e-5), N.NS_BF16, dyb.ptr, 0)
    dev.synchronize()
    assert orc.close(s_exp, ds.download(), 1e-2)
    dq_h = dq.download((rows, cols)).astype(np.int32)
    diff = np.abs(dq_h - q_exp.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    assert orc.close(expb, orc.widen_bf16(dyb.download((rows, cols))), 1e-2)


def test_embed_argmax_counter(dev, orc):
    V, D, ctx, B, T = 50, 64, 32, 3, 4
    tok = orc.round_bf16(orc.normal((V, D), 101, 0.02))
    pos = orc.round_bf16(orc.normal((ctx, D), 102, 0.02))
    ids = np.array(orc.token_ids((B, T), 103, V), np.int32)
    dtok, dpos, dids = dev.from_numpy(tok), dev.from_numpy(pos), dev.from_numpy(ids)
    dp = dev.from_numpy(np.array([5], np.int32))
    dy = dev.empty(B * T * D, N.NS_BF16)
    N.call("ns_embed_pos", dev.handle, dids.ptr, dtok.ptr, dpos.ptr, N.NS_BF16, dp.ptr, B, T, D, V, ctx, N.NS_BF16, dy.ptr)
    N.call("ns_add_i32", dev.handle, dp.ptr, T)
    dev.synchronize()
    exp = orc.widen_bf16(tok)[ids] + orc.widen_bf16(pos)[5:5 + T][None]
    assert np.array_equal(orc.round_bf16(exp), dy.download((B, T, D)))
    assert dp.download()[0] == 9
    x = orc.normal((5, 32000), 104)
    x[1, 31999] = 50.0
    x[2, [7, 20000]] = 60.0
    dx, di = dev.from_numpy(x), dev.empty(5, N.NS_I32)
    N.call("ns_argmax_i32", dev.handle, dx.ptr, 5, 32000, C.c_int64(32000), di.ptr)
    dev.synchronize()
    assert np.array_equal(orc.argmax(x).astype(np.int32), di.download())


def test_a_second_stream_waits_for_an_event_of_the_first(dev):
    """Two device objects on one GPU are two streams.  The first fills 256 MB several times over and records an event; the
    second waits for the event (ns_stream_wait_event) and copies the buffer: the copy must hold the last fill, every time."""
    from nn_b200.device import Device
    side = Device(dev.ordinal)
    try:
        n = 64 * 1024 * 1024
        a, b = dev.empty(n), dev.empty(n)
        ev = dev.event()
        for rep in range(3):
            for seed in range(4):      # keep the first stream busy, the last fill is the one that counts
                N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_F32, C.c_int64(n), 100 + 10 * rep + seed, C.c_float(0.0), C.c_float(1.0))
            dev.record(ev)
            side.wait_event(ev)
            N.call("ns_d2d_async", side.handle, C.c_uint64(b.ptr), C.c_uint64(a.ptr), C.c_uint64(4 * n))
            side.synchronize()
            dev.synchronize()
            got, want = b.download(count=4096, offset=n - 4096), a.download(count=4096, offset=n - 4096)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"repetition {rep}"
    finally:
        side.close()


def test_many_row_kernel_gives_up_when_a_copy_never_arrives(dev, orc):
    """Failure detection without a GPU fault: the test hook makes the many-row quantisation leave out the copy of one row.  The
    warp that owns the row waits for it, gives up after about a second, reports status 600 + warps per row through the next
    synchronisation (NS_ERR_KERNEL), waits once more for what it still has in flight and returns; the other rows are
    finished, and the device stays usable."""
    rows, cols = 4096, 2048
    x = orc.round_bf16(orc.normal((rows, cols), 99, 1.5))
    dx = dev.from_numpy(x)
    dq, ds = dev.zeros(rows * cols, N.NS_I8), dev.zeros(rows)
    dev.tune(600, 5)          # NS_TUNE_DROP_ROW: the copy of row 5 is left out
    try:
        N.call("ns_quantize_rows_i8", dev.handle, dx.ptr, N.NS_BF16, C.c_int64(rows), cols, dq.ptr, ds.ptr)
        with pytest.raises(N.NsError) as err:
            dev.synchronize()
        assert "status 601" in str(err.value)
    finally:
        dev.tune(0, 0)
    q, sc = orc.quantize_rows_i8(x)
    got = dq.download((rows, cols))
    assert not got[5].any(), "the row whose copy never came must not be written"
    done = np.abs(got).max(axis=1) > 0                     # (no row of this input quantises to all zeros)
    assert done.sum() >= rows - 8 and not done[5], "only rows of the group that gave up may be missing"
    assert np.array_equal(got[done], q[done])
    # the device is still usable
    N.call("ns_quantize_rows_i8", dev.handle, dx.ptr, N.NS_BF16, C.c_int64(rows), cols, dq.ptr, ds.ptr)
    dev.synchronize()
    assert np.array_equal(dq.download((rows, cols)), q) and np.array_equal(ds.download(), sc)
