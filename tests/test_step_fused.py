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


def test_fused_and_unfused_decoder_agree(dev, orc):
    """The int8 decoder with and without the fused row kernels: same tokens, bit-identical logits (head_dim 64, so both
    variants read the few prompt rows with the decode attention kernel)."""
    from nn_b200.gpt import GptConfig, GptW8A8
    from oracle import model as om
    cfg = GptConfig(vocab=320, dim=256, heads=4, layers=3, ff_dim=1024, context=48)
    w = om.make_weights(cfg, seed=6)
    prompt = orc.token_ids((4, 9), 3, cfg.vocab).astype(np.int64)
    out = []
    for fused in (True, False):
        m = GptW8A8(dev, cfg, w, 4, max_prefill=16)
        m.fused = fused
        tokens, _ = m.generate(prompt, 20, use_graph=True)
        dev.synchronize()
        out.append((np.asarray(tokens), m.read_logits()))
        m.close()
    assert np.array_equal(out[0][0], out[1][0])
    assert np.array_equal(out[0][1].view(np.uint32), out[1][1].view(np.uint32))



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
