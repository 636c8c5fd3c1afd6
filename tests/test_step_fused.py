"""Fused row kernels of the decoding step (ns_linear_forward_partial + ns_finish_norm_quant / ns_finish_kv_append).

They must give, bit for bit, what the unfused sequence gives (product with its own epilogue, then ns_layernorm with int8
output / ns_kv_append), which the other tests hold to the oracle; and directly the oracle's W8A8 Linear + residual.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


def _linear(dev, w_kn, bias):
    h = C.c_void_p()
    w = np.ascontiguousarray(w_kn, np.float32)
    b = np.ascontiguousarray(bias, np.float32)
    N.call("ns_linear_create", dev.handle, w.shape[0], w.shape[1], N.NS_I8, w.ctypes.data_as(C.POINTER(C.c_float)),
           b.ctypes.data_as(C.POINTER(C.c_float)), N.SPLIT_NONE, 1, 0, 1, C.byref(h))
    return h


def _partial(dev, lin, xq, m):
    ptr, sp = C.c_uint64(), C.c_int()
    N.call("ns_linear_forward_partial", dev.handle, lin, C.c_uint64(xq.ptr), m, C.byref(ptr), C.byref(sp))
    return ptr.value, sp.value


@pytest.mark.parametrize("M,K,NN,tune", [(64, 2048, 2048, (0, 0)), (64, 8192, 2048, (0, 0)), (3, 256, 128, (0, 0)), (64, 2048, 2048, (128, 1)),
                                         (17, 1024, 520, (64, 3)), (200, 512, 1024, (0, 0))])
def test_finish_norm_quant_equals_unfused(dev, orc, M, K, NN, tune):
    x = orc.normal((M, K), 5)
    w = orc.normal((K, NN), 6, 0.05)
    bias = orc.normal((NN,), 7, 0.1)
    res = orc.round_bf16(orc.normal((M, NN), 8))
    gamma, beta = (1.0 + orc.normal((NN,), 9, 0.1)).astype(np.float32), orc.normal((NN,), 10, 0.1)
    lin = _linear(dev, w, bias)
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    d_res, d_g, d_b = dev.from_numpy(res), dev.from_numpy(gamma), dev.from_numpy(beta)
    # unfused: product with bias + residual epilogue -> bf16, then LayerNorm -> int8
    y_ref, q_ref, s_ref = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
    dev.tune(*tune)
    try:
        N.call("ns_linear_forward", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), M, N.EPI_BIAS_RESIDUAL, C.c_uint64(d_res.ptr), N.NS_BF16,
               N.NS_BF16, C.c_uint64(y_ref.ptr))
        N.call("ns_layernorm", dev.handle, y_ref.ptr, N.NS_BF16, d_g.ptr, d_b.ptr, C.c_int64(M), NN, C.c_float(1e-5), N.NS_I8, q_ref.ptr, s_ref.ptr)
        # fused; q_scale written over the array the input scales were read from, as the decoder does
        part, sp = _partial(dev, lin, xq, M)
    finally:
        dev.tune(0, 0)
    y, q, s = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), xs
    N.call("ns_finish_norm_quant", dev.handle, C.c_uint64(part), sp, lin, xs.ptr, d_res.ptr, C.c_int64(M), y.ptr, d_g.ptr, d_b.ptr, C.c_float(1e-5),
           q.ptr, s.ptr)
    dev.synchronize()
    assert np.array_equal(y.download(), y_ref.download())
    assert np.array_equal(q.download(), q_ref.download())
    assert np.array_equal(s.download().view(np.uint32), s_ref.download().view(np.uint32))
    # and the oracle's Linear + residual directly
    oq, osc = orc.quantize_rows_i8(x)
    wq, ws = orc.quantize_rows_i8(np.ascontiguousarray(w.T))
    exp = orc.dequant_epilogue(orc.qmatmul_i8_acc(oq, wq), osc, ws, bias=bias, residual=orc.widen_bf16(res))
    assert np.array_equal(y.download((M, NN)), orc.round_bf16(exp))
    # without LayerNorm: only the residual stream is written
    y2 = dev.empty(M * NN, N.NS_BF16)
    xs2 = dev.from_numpy(osc)
    part, sp = _partial(dev, lin, xq, M)
    N.call("ns_finish_norm_quant", dev.handle, C.c_uint64(part), sp, lin, xs2.ptr, d_res.ptr, C.c_int64(M), y2.ptr, 0, 0, C.c_float(1e-5), 0, 0)
    dev.synchronize()
    assert np.array_equal(y2.download(), y_ref.download())
    N.call("ns_linear_destroy", lin)


@pytest.mark.parametrize("B,steps,heads,dh,pos0", [(64, 1, 16, 128, 37), (3, 2, 4, 32, 0), (5, 1, 2, 64, 63)])
def test_finish_kv_append_equals_unfused(dev, orc, B, steps, heads, dh, pos0):
    D = heads * dh
    K, NN, M = 256, 3 * heads * dh, B * steps
    x = orc.normal((M, K), 15)
    w = orc.normal((K, NN), 16, 0.05)
    bias = orc.normal((NN,), 17, 0.1)
    lin = _linear(dev, w, bias)
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    page_size, max_pages = 16, 8
    table = dev.from_numpy(np.random.default_rng(1).permutation(B * max_pages).astype(np.int32))
    pos = dev.from_numpy(np.array([pos0], np.int32))
    pools = []
    qkvs = []
    for fused in (False, True):
        cache = C.c_void_p()
        N.call("ns_kv_cache_create", dev.handle, B * max_pages, page_size, heads, dh, C.byref(cache))
        qkv = dev.zeros(M * NN, N.NS_BF16)
        if fused:
            part, sp = _partial(dev, lin, xq, M)
            N.call("ns_finish_kv_append", dev.handle, C.c_uint64(part), sp, lin, xs.ptr, B, steps, qkv.ptr, cache, table.ptr, max_pages, pos.ptr)
        else:
            N.call("ns_linear_forward", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), M, N.EPI_BIAS, C.c_uint64(0), N.NS_BF16, N.NS_BF16,
                   C.c_uint64(qkv.ptr))
            N.call("ns_kv_append", dev.handle, cache, C.c_uint64(qkv.ptr + 2 * D), C.c_uint64(qkv.ptr + 4 * D), C.c_int64(NN), table.ptr, max_pages,
                   pos.ptr, B, steps)
        dev.synchronize()
        kp, vp, nbytes = C.c_uint64(), C.c_uint64(), C.c_uint64()
        N.call("ns_kv_cache_pools", cache, C.byref(kp), C.byref(vp), C.byref(nbytes))
        host = np.empty((2, nbytes.value // 2), np.uint16)
        N.call("ns_d2h", dev.handle, host[0].ctypes.data_as(C.c_void_p), kp, nbytes)
        N.call("ns_d2h", dev.handle, host[1].ctypes.data_as(C.c_void_p), vp, nbytes)
        pools.append(host)
        qkvs.append(qkv.download())
        N.call("ns_kv_cache_destroy", cache)
    assert np.array_equal(qkvs[0], qkvs[1])
    assert np.array_equal(pools[0], pools[1])
    assert pools[1].any(), "something must have been appended"
    N.call("ns_linear_destroy", lin)


@pytest.mark.parametrize("dim,heads,ff", [(256, 4, 1024), (768, 12, 1536)])
def test_fused_and_unfused_decoder_agree(dev, orc, dim, heads, ff):
    """The int8 decoder with one launch per Linear (2), with the fused row kernels (1) and with one kernel per operator
    (0): same tokens, bit-identical logits (head_dim 64, so every variant reads the few prompt rows with the decode
    attention kernel; with head_dim 128 the unfused variant would take the flash kernel, which rounds P to bf16)."""
    from nn_b200.gpt import GptConfig, GptW8A8
    from oracle import model as om
    cfg = GptConfig(vocab=320, dim=dim, heads=heads, layers=3, ff_dim=ff, context=48)
    w = om.make_weights(cfg, seed=6)
    prompt = orc.token_ids((4, 9), 3, cfg.vocab).astype(np.int64)
    out = []
    for fused in (2, 1, 0):
        m = GptW8A8(dev, cfg, w, 4, max_prefill=16)
        m.fused = fused
        tokens, _ = m.generate(prompt, 20, use_graph=True)
        dev.synchronize()
        out.append((np.asarray(tokens), m.read_logits(), m.launches_per_step))
        m.close()
    for other in out[1:]:
        assert np.array_equal(out[0][0], other[0])
        assert np.array_equal(out[0][1].view(np.uint32), other[1].view(np.uint32))
    assert out[0][2] < out[1][2] <= out[2][2], "one launch per Linear must take fewer launches per step (split-K second kernels are not counted)"



@pytest.mark.parametrize("M,NN", [(64, 2048), (5, 256), (200, 1024)])
def test_peer_reduce_single_rank_equals_unfused(dev, orc, M, NN):
    """ns_tp_reduce_norm_quant with one rank (the sum over ranks is the rank's own slot): bias + residual, LayerNorm and
    quantisation must equal ns_bias_residual followed by ns_layernorm bit for bit, call after call (the epoch of a slot
    advances on the device), and for both slots."""
    group = C.c_void_p()
    N.call("ns_peer_group_create", dev.handle, 0, 1, C.c_uint64(256 * 8192 * 4), C.byref(group))
    bias = orc.normal((NN,), 31, 0.1)
    gamma, beta = (1.0 + orc.normal((NN,), 32, 0.1)).astype(np.float32), orc.normal((NN,), 33, 0.1)
    d_bias, d_g, d_b = dev.from_numpy(bias), dev.from_numpy(gamma), dev.from_numpy(beta)
    for call in range(3):
        slot = call & 1
        part = orc.normal((M, NN), 40 + call)
        res = orc.round_bf16(orc.normal((M, NN), 50 + call))
        ptr = C.c_uint64()
        N.call("ns_peer_group_slot", group, slot, C.byref(ptr))
        N.call("ns_h2d", dev.handle, ptr, part.ctypes.data_as(C.c_void_p), C.c_uint64(part.nbytes))
        d_part, d_res = dev.from_numpy(part), dev.from_numpy(res)
        y_ref, q_ref, s_ref = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
        N.call("ns_bias_residual", dev.handle, C.c_uint64(d_part.ptr), C.c_uint64(d_bias.ptr), C.c_uint64(d_res.ptr), N.NS_BF16, C.c_int64(M), NN,
               N.NS_BF16, C.c_uint64(y_ref.ptr))
        N.call("ns_layernorm", dev.handle, y_ref.ptr, N.NS_BF16, d_g.ptr, d_b.ptr, C.c_int64(M), NN, C.c_float(1e-5), N.NS_I8, q_ref.ptr, s_ref.ptr)
        y, q, s = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
        N.call("ns_tp_reduce_norm_quant", dev.handle, group, slot, C.c_uint64(d_bias.ptr), d_res.ptr, C.c_int64(M), NN, y.ptr, d_g.ptr, d_b.ptr,
               C.c_float(1e-5), q.ptr, s.ptr)
        dev.synchronize()
        assert np.array_equal(y.download(), y_ref.download())
        assert np.array_equal(q.download(), q_ref.download())
        assert np.array_equal(s.download().view(np.uint32), s_ref.download().view(np.uint32))
    N.call("ns_peer_group_destroy", group)


def test_peer_reduce_gives_up_when_a_rank_never_arrives(dev, orc):
    """Failure detection without a GPU fault: a group of two whose second rank is a stand-in that never signals.  The
    kernel's wait runs out (about a second), the next synchronisation reports NS_ERR_KERNEL with status 400 + the missing
    rank, and the device stays usable: a complete group of one works right afterwards."""
    M, NN = 8, 256
    group = C.c_void_p()
    N.call("ns_peer_group_create", dev.handle, 0, 2, C.c_uint64(256 * 1024), C.byref(group))
    N.call("ns_peer_group_connect", group, None)
    y = dev.zeros(M * NN, N.NS_BF16)
    N.call("ns_tp_reduce_norm_quant", dev.handle, group, 0, C.c_uint64(0), 0, C.c_int64(M), NN, y.ptr, 0, 0, C.c_float(1e-5), 0, 0)
    with pytest.raises(N.NsError) as err:
        dev.synchronize()
    assert "status 401" in str(err.value)
    assert not y.download().any(), "no row may be written when a rank is missing"
    N.call("ns_peer_group_destroy", group)
    # the device is still usable
    solo = C.c_void_p()
    N.call("ns_peer_group_create", dev.handle, 0, 1, C.c_uint64(256 * 1024), C.byref(solo))
    part = orc.normal((M, NN), 3)
    ptr = C.c_uint64()
    N.call("ns_peer_group_slot", solo, 0, C.byref(ptr))
    N.call("ns_h2d", dev.handle, ptr, part.ctypes.data_as(C.c_void_p), C.c_uint64(part.nbytes))
    N.call("ns_tp_reduce_norm_quant", dev.handle, solo, 0, C.c_uint64(0), 0, C.c_int64(M), NN, y.ptr, 0, 0, C.c_float(1e-5), 0, 0)
    dev.synchronize()
    assert np.array_equal(y.download((M, NN)), orc.round_bf16(part))
    N.call("ns_peer_group_destroy", solo)


# ---------------------------------------------------------------------------------------------------------------
# one launch per Linear: the product kernel's second phase (ns_linear_forward_norm_quant / _gelu_quant / _kv_append)
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,NN,tune", [(64, 2048, 2048, (0, 0)), (64, 8192, 2048, (0, 0)), (3, 256, 256, (0, 0)), (64, 2048, 2048, (128, 1)),
                                         (17, 1024, 768, (64, 3)), (200, 512, 1024, (0, 0)), (256, 1024, 8192, (0, 0)), (64, 2048, 4096, (256, 2))])
def test_one_launch_norm_quant_equals_two_launches(dev, orc, M, K, NN, tune):
    x = orc.normal((M, K), 5)
    w = orc.normal((K, NN), 6, 0.05)
    bias = orc.normal((NN,), 7, 0.1)
    res = orc.round_bf16(orc.normal((M, NN), 8))
    gamma, beta = (1.0 + orc.normal((NN,), 9, 0.1)).astype(np.float32), orc.normal((NN,), 10, 0.1)
    lin = _linear(dev, w, bias)
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    d_res, d_g, d_b = dev.from_numpy(res), dev.from_numpy(gamma), dev.from_numpy(beta)
    y_ref, q_ref, s_ref = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
    dev.tune(*tune)
    try:
        part, sp = _partial(dev, lin, xq, M)
        N.call("ns_finish_norm_quant", dev.handle, C.c_uint64(part), sp, lin, xs.ptr, d_res.ptr, C.c_int64(M), y_ref.ptr, d_g.ptr, d_b.ptr,
               C.c_float(1e-5), q_ref.ptr, s_ref.ptr)
        dev.synchronize()
        for rep in range(3):      # the arrival counters must be back at zero after every launch
            y, q, s = dev.zeros(M * NN, N.NS_BF16), dev.zeros(M * NN, N.NS_I8), dev.zeros(M)
            N.call("ns_linear_forward_norm_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), d_res.ptr, C.c_int64(M), y.ptr, d_g.ptr,
                   d_b.ptr, C.c_float(1e-5), q.ptr, s.ptr)
            dev.synchronize()
            assert np.array_equal(y.download(), y_ref.download()), f"repetition {rep}"
            assert np.array_equal(q.download(), q_ref.download()), f"repetition {rep}"
            assert np.array_equal(s.download().view(np.uint32), s_ref.download().view(np.uint32)), f"repetition {rep}"
        # without LayerNorm: only the residual stream is written; and q_scale written over the array x_scale is read from
        y2 = dev.zeros(M * NN, N.NS_BF16)
        N.call("ns_linear_forward_norm_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), d_res.ptr, C.c_int64(M), y2.ptr, 0, 0,
               C.c_float(1e-5), 0, 0)
        q3 = dev.zeros(M * NN, N.NS_I8)
        N.call("ns_linear_forward_norm_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), d_res.ptr, C.c_int64(M), y.ptr, d_g.ptr,
               d_b.ptr, C.c_float(1e-5), q3.ptr, xs.ptr)
        dev.synchronize()
    finally:
        dev.tune(0, 0)
    assert np.array_equal(y2.download(), y_ref.download())
    assert np.array_equal(q3.download(), q_ref.download())
    assert np.array_equal(xs.download().view(np.uint32), s_ref.download().view(np.uint32))
    N.call("ns_linear_destroy", lin)


@pytest.mark.parametrize("M,K,NN,tune", [(64, 2048, 8192, (0, 0)), (64, 2048, 4096, (0, 0)), (5, 256, 1024, (0, 0)), (200, 512, 2048, (128, 2)),
                                         (64, 1024, 1024, (64, 1))])
def test_one_launch_gelu_quant_equals_two_launches(dev, orc, M, K, NN, tune):
    x = orc.normal((M, K), 25)
    w = orc.normal((K, NN), 26, 0.05)
    bias = orc.normal((NN,), 27, 0.1)
    lin = _linear(dev, w, bias)
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    hid, q_ref, s_ref = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
    dev.tune(*tune)
    try:
        N.call("ns_linear_forward", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), M, N.EPI_BIAS_GELU, C.c_uint64(0), N.NS_BF16, N.NS_BF16,
               C.c_uint64(hid.ptr))
        N.call("ns_quantize_rows_i8", dev.handle, hid.ptr, N.NS_BF16, C.c_int64(M), NN, q_ref.ptr, s_ref.ptr)
        for rep in range(2):
            q, s = dev.zeros(M * NN, N.NS_I8), dev.zeros(M)
            N.call("ns_linear_forward_gelu_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), C.c_int64(M), q.ptr, s.ptr)
            dev.synchronize()
            assert np.array_equal(q.download(), q_ref.download()), f"repetition {rep}"
            assert np.array_equal(s.download().view(np.uint32), s_ref.download().view(np.uint32)), f"repetition {rep}"
        # the two-launch form of the decoding step: partial sums, then one row kernel for sum + bias + GELU + quantisation
        q2, s2 = dev.zeros(M * NN, N.NS_I8), dev.zeros(M)
        part, sp = _partial(dev, lin, xq, M)
        N.call("ns_finish_gelu_quant", dev.handle, C.c_uint64(part), sp, lin, xs.ptr, C.c_int64(M), q2.ptr, s2.ptr)
        dev.synchronize()
        assert np.array_equal(q2.download(), q_ref.download())
        assert np.array_equal(s2.download().view(np.uint32), s_ref.download().view(np.uint32))
    finally:
        dev.tune(0, 0)
    N.call("ns_linear_destroy", lin)


@pytest.mark.parametrize("B,steps,heads,dh,pos0", [(64, 1, 16, 128, 37), (3, 2, 4, 32, 0), (5, 1, 2, 64, 63), (64, 1, 2, 128, 600), (12, 1, 2, 128, 40),
                                                  (4, 3, 2, 64, 5), (16, 1, 4, 128, 0), (1, 1, 2, 128, 9), (8, 1, 16, 128, 100)])
def test_one_launch_kv_append_equals_unfused(dev, orc, B, steps, heads, dh, pos0):
    D = heads * dh
    K, NN, M = 256, 3 * heads * dh, B * steps
    x = orc.normal((M, K), 15)
    w = orc.normal((K, NN), 16, 0.05)
    bias = orc.normal((NN,), 17, 0.1)
    lin = _linear(dev, w, bias)
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    page_size, max_pages = 16, (pos0 + steps) // 16 + 1
    table = dev.from_numpy(np.random.default_rng(1).permutation(B * max_pages).astype(np.int32))
    pos = dev.from_numpy(np.array([pos0], np.int32))
    pools, qkvs = [], []
    for fused in (False, True):
        cache = C.c_void_p()
        N.call("ns_kv_cache_create", dev.handle, B * max_pages, page_size, heads, dh, C.byref(cache))
        qkv = dev.zeros(M * NN, N.NS_BF16)
        if fused:
            N.call("ns_linear_forward_kv_append", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), B, steps, qkv.ptr, cache, table.ptr,
                   max_pages, pos.ptr)
        else:
            N.call("ns_linear_forward", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), M, N.EPI_BIAS, C.c_uint64(0), N.NS_BF16, N.NS_BF16,
                   C.c_uint64(qkv.ptr))
            N.call("ns_kv_append", dev.handle, cache, C.c_uint64(qkv.ptr + 2 * D), C.c_uint64(qkv.ptr + 4 * D), C.c_int64(NN), table.ptr, max_pages,
                   pos.ptr, B, steps)
        dev.synchronize()
        kp, vp, nbytes = C.c_uint64(), C.c_uint64(), C.c_uint64()
        N.call("ns_kv_cache_pools", cache, C.byref(kp), C.byref(vp), C.byref(nbytes))
        host = np.empty((2, nbytes.value // 2), np.uint16)
        N.call("ns_d2h", dev.handle, host[0].ctypes.data_as(C.c_void_p), kp, nbytes)
        N.call("ns_d2h", dev.handle, host[1].ctypes.data_as(C.c_void_p), vp, nbytes)
        pools.append(host)
        qkvs.append(qkv.download())
        N.call("ns_kv_cache_destroy", cache)
    assert np.array_equal(qkvs[0], qkvs[1])
    assert np.array_equal(pools[0], pools[1])
    assert pools[1].any(), "something must have been appended"
    N.call("ns_linear_destroy", lin)


@pytest.mark.parametrize("B,heads,dh,length", [(64, 16, 128, 300), (64, 2, 128, 700), (5, 4, 64, 90), (3, 8, 32, 40)])
def test_attention_decode_quant_equals_attention_then_quantise(dev, orc, B, heads, dh, length):
    """The attention kernel's last CTA per output row quantises the row (with and without a split cache)."""
    page_size = 16
    max_pages = (length + page_size) // page_size
    cache = C.c_void_p()
    N.call("ns_kv_cache_create", dev.handle, B * max_pages, page_size, heads, dh, C.byref(cache))
    kp, vp, nbytes = C.c_uint64(), C.c_uint64(), C.c_uint64()
    N.call("ns_kv_cache_pools", cache, C.byref(kp), C.byref(vp), C.byref(nbytes))
    N.call("ns_fill_normal", dev.handle, kp, N.NS_BF16, C.c_int64(nbytes.value // 2), 2, C.c_float(0.0), C.c_float(1.0))
    N.call("ns_fill_normal", dev.handle, vp, N.NS_BF16, C.c_int64(nbytes.value // 2), 3, C.c_float(0.0), C.c_float(1.0))
    table = dev.from_numpy(np.random.default_rng(2).permutation(B * max_pages).astype(np.int32))
    pos = dev.from_numpy(np.array([length - 1], np.int32))
    D = heads * dh
    q = dev.from_numpy(orc.round_bf16(orc.normal((B, D), 71)))
    o_ref, q_ref, s_ref = dev.empty(B * D, N.NS_BF16), dev.empty(B * D, N.NS_I8), dev.empty(B)
    scale = C.c_float(1.0 / np.sqrt(dh))
    N.call("ns_attention_decode", dev.handle, cache, q.ptr, C.c_int64(D), o_ref.ptr, C.c_int64(D), table.ptr, max_pages, pos.ptr, B, 1, scale)
    N.call("ns_quantize_rows_i8", dev.handle, o_ref.ptr, N.NS_BF16, C.c_int64(B), D, q_ref.ptr, s_ref.ptr)
    for rep in range(2):
        o, qq, ss = dev.zeros(B * D, N.NS_BF16), dev.zeros(B * D, N.NS_I8), dev.zeros(B)
        N.call("ns_attention_decode_quant", dev.handle, cache, q.ptr, C.c_int64(D), o.ptr, C.c_int64(D), table.ptr, max_pages, pos.ptr, B, 1, scale,
               qq.ptr, ss.ptr)
        dev.synchronize()
        assert np.array_equal(o.download(), o_ref.download()), f"repetition {rep}"
        assert np.array_equal(qq.download(), q_ref.download()), f"repetition {rep}"
        assert np.array_equal(ss.download().view(np.uint32), s_ref.download().view(np.uint32)), f"repetition {rep}"
    N.call("ns_kv_cache_destroy", cache)


@pytest.mark.parametrize("M,K,NN", [(64, 1024, 2048), (5, 256, 256), (128, 512, 1024)])
def test_one_launch_peer_exchange_single_rank(dev, orc, M, K, NN):
    """ns_linear_forward_tp_norm_quant with a group of one: the product, the arrival counter, the flag raised for this
    rank itself and the row pass -- against ns_linear_forward into the slot followed by ns_tp_reduce_norm_quant."""
    x = orc.normal((M, K), 81)
    w = orc.normal((K, NN), 82, 0.05)
    bias = orc.normal((NN,), 83, 0.1)
    res = orc.round_bf16(orc.normal((M, NN), 84))
    gamma, beta = (1.0 + orc.normal((NN,), 85, 0.1)).astype(np.float32), orc.normal((NN,), 86, 0.1)
    h = C.c_void_p()
    wc, bc = np.ascontiguousarray(w, np.float32), np.ascontiguousarray(bias, np.float32)
    # a row shard of a one-rank group: same weights, the layer keeps its bias for after the exchange
    N.call("ns_linear_create", dev.handle, K, NN, N.NS_I8, wc.ctypes.data_as(C.POINTER(C.c_float)), bc.ctypes.data_as(C.POINTER(C.c_float)),
           N.SPLIT_ROW, 1, 0, 1, C.byref(h))
    bias_ptr = C.c_uint64()
    N.call("ns_linear_info", h, None, None, None, None, None, C.byref(bias_ptr))
    group = C.c_void_p()
    N.call("ns_peer_group_create", dev.handle, 0, 1, C.c_uint64(256 * 8192 * 4), C.byref(group))
    d_x = dev.from_numpy(x)
    xq, xs = dev.empty(M * K, N.NS_I8), dev.empty(M)
    N.call("ns_quantize_rows_i8", dev.handle, d_x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
    d_res, d_g, d_b = dev.from_numpy(res), dev.from_numpy(gamma), dev.from_numpy(beta)
    for call in range(4):
        slot = call & 1
        ptr = C.c_uint64()
        N.call("ns_peer_group_slot", group, slot, C.byref(ptr))
        y_ref, q_ref, s_ref = dev.empty(M * NN, N.NS_BF16), dev.empty(M * NN, N.NS_I8), dev.empty(M)
        N.call("ns_linear_forward", dev.handle, h, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), M, N.EPI_NONE, C.c_uint64(0), N.NS_BF16, N.NS_F32, ptr)
        N.call("ns_tp_reduce_norm_quant", dev.handle, group, slot, bias_ptr, d_res.ptr, C.c_int64(M), NN, y_ref.ptr, d_g.ptr, d_b.ptr,
               C.c_float(1e-5), q_ref.ptr, s_ref.ptr)
        dev.synchronize()
        N.call("ns_memset32_async", dev.handle, ptr, 0, C.c_uint64(M * NN))
        y, q, s = dev.zeros(M * NN, N.NS_BF16), dev.zeros(M * NN, N.NS_I8), dev.zeros(M)
        N.call("ns_linear_forward_tp_norm_quant", dev.handle, h, group, slot, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), d_res.ptr, C.c_int64(M), y.ptr,
               d_g.ptr, d_b.ptr, C.c_float(1e-5), q.ptr, s.ptr)
        dev.synchronize()
        assert np.array_equal(y.download(), y_ref.download()), f"call {call}"
        assert np.array_equal(q.download(), q_ref.download()), f"call {call}"
        assert np.array_equal(s.download().view(np.uint32), s_ref.download().view(np.uint32)), f"call {call}"
    N.call("ns_peer_group_destroy", group)
    N.call("ns_linear_destroy", h)
