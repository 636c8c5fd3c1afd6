"""Causal attention over a whole sequence (ns_attention_prefill, tcgen05) against the oracle's reference-order
attention: scale, additive mask, row maximum, exp, float sum, normalise, . V (Layers/Attention.cs:54-90,
CpuBackend.Decoding.cs:9-41) on the same bf16-rounded inputs.  Tolerance 1e-2 relative on bf16 outputs.
benchmark configuration 4: [batch 8, heads 32, seq, 128], seq in {512, 2048, 8192}, scale 1/sqrt(128), seed 3.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu
TOL = 1e-2
DH = 128


def _strides(*v):
    return (C.c_int64 * 3)(*v)


def _run_bhsd(dev, q, k, v, B, H, S, scale, causal=True):
    dq, dk, dv = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v)
    do = dev.zeros(B * H * S * DH, N.NS_BF16)
    st = _strides(H * S * DH, S * DH, DH)
    N.call("ns_attention_prefill", dev.handle, dq.ptr, dk.ptr, dv.ptr, do.ptr, B, H, S, DH, st, st, st, st, C.c_float(scale), int(causal))
    dev.synchronize()
    return do.download((B, H, S, DH))


@pytest.mark.parametrize("S", [1, 37, 128, 129, 300, 640])
@pytest.mark.parametrize("causal", [True, False])
def test_small_sequences(dev, orc, S, causal):
    B, H = 2, 3
    scale = 1.0 / np.sqrt(DH)
    q = orc.round_bf16(orc.normal((B, H, S, DH), 1))
    k = orc.round_bf16(orc.normal((B, H, S, DH), 2))
    v = orc.round_bf16(orc.normal((B, H, S, DH), 3))
    got = orc.widen_bf16(_run_bhsd(dev, q, k, v, B, H, S, scale, causal))
    for b in range(B):
        for h in range(H):
            exp = orc.attention_slice(orc.widen_bf16(q[b, h]), orc.widen_bf16(k[b, h]), orc.widen_bf16(v[b, h]), 0, scale, causal)
            assert orc.close(orc.bf16_round_trip(exp), got[b, h], TOL), (b, h, orc.max_err(exp, got[b, h]))


def test_large_scores_and_growing_maximum(dev, orc):
    """Scores that keep growing along the sequence force the running maximum (and the rescale of O) to move."""
    B, H, S = 1, 2, 512
    q = orc.normal((B, H, S, DH), 4)
    k = orc.normal((B, H, S, DH), 5)
    k *= np.linspace(0.2, 6.0, S, dtype=np.float32)[None, None, :, None]
    v = orc.normal((B, H, S, DH), 6)
    qb, kb, vb = orc.round_bf16(q), orc.round_bf16(k), orc.round_bf16(v)
    scale = 0.5
    got = orc.widen_bf16(_run_bhsd(dev, qb, kb, vb, B, H, S, scale))
    for h in range(H):
        exp = orc.attention_slice(orc.widen_bf16(qb[0, h]), orc.widen_bf16(kb[0, h]), orc.widen_bf16(vb[0, h]), 0, scale)
        assert orc.close(orc.bf16_round_trip(exp), got[0, h], TOL), orc.max_err(exp, got[0, h])


def test_fused_qkv_layout(dev, orc):
    """q, k, v read in place from a [batch * seq, 3 * D] buffer (the output of the fused QKV product), o written
    as [batch * seq, D]: the reference's narrow + permute copies (Attention.cs:54-58) are not needed."""
    B, H, S = 2, 4, 200
    D = H * DH
    scale = 1.0 / np.sqrt(DH)
    qkv = orc.round_bf16(orc.normal((B, S, 3 * D), 7))
    dqkv = dev.from_numpy(qkv)
    do = dev.zeros(B * S * D, N.NS_BF16)
    st_in = _strides(S * 3 * D, DH, 3 * D)
    st_out = _strides(S * D, DH, D)
    N.call("ns_attention_prefill", dev.handle, dqkv.ptr, dqkv.ptr + 2 * D, dqkv.ptr + 4 * D, do.ptr, B, H, S, DH, st_in, st_in, st_in, st_out,
           C.c_float(scale), 1)
    dev.synchronize()
    got = orc.widen_bf16(do.download((B, S, H, DH)))
    f = orc.widen_bf16(qkv).reshape(B, S, 3, H, DH)
    for b in range(B):
        for h in range(H):
            exp = orc.attention_slice(f[b, :, 0, h], f[b, :, 1, h], f[b, :, 2, h], 0, scale)
            assert orc.close(orc.bf16_round_trip(exp), got[b, :, h], TOL), (b, h, orc.max_err(exp, got[b, :, h]))


@pytest.mark.parametrize("S", [512, 2048, 8192])
def test_baseline_shapes(dev, orc, S):
    B, H = 8, 32
    scale = 1.0 / np.sqrt(DH)
    n = B * H * S * DH
    dq, dk, dv, do = (dev.empty(n, N.NS_BF16) for _ in range(4))
    for t, seed in ((dq, 31), (dk, 32), (dv, 33)):
        N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_BF16, C.c_int64(n), seed, C.c_float(0.0), C.c_float(1.0))
    st = _strides(H * S * DH, S * DH, DH)
    N.call("ns_attention_prefill", dev.handle, dq.ptr, dk.ptr, dv.ptr, do.ptr, B, H, S, DH, st, st, st, st, C.c_float(scale), 1)
    dev.synchronize()
    rng = np.random.default_rng(S)
    for (b, h) in [(0, 0), (7, 31), (3, 17)]:
        off = (b * H + h) * S * DH
        qs, ks, vs, os_ = (orc.widen_bf16(t.download((S, DH), offset=off, count=S * DH)) for t in (dq, dk, dv, do))
        starts = sorted(set([0, S - 64, S // 2 - 32] + [int(x) for x in rng.integers(0, S - 64, 2)]))
        for r0 in starts:
            exp = orc.attention_slice(qs[r0:r0 + 64], ks, vs, r0, scale)
            assert orc.close(orc.bf16_round_trip(exp), os_[r0:r0 + 64], TOL), (b, h, r0, orc.max_err(exp, os_[r0:r0 + 64]))
    # size-independent property: row 0 attends to key 0 only, so o[:, :, 0, :] == v[:, :, 0, :] exactly
    o0 = do.download((B * H, S * DH))[:, :DH]
    v0 = dv.download((B * H, S * DH))[:, :DH]
    assert np.array_equal(o0, v0)


def test_results_do_not_depend_on_the_tile_schedule(dev, orc):
    """The kernel's CTAs draw their (batch, head, query tile) work from a counter at run time, so which CTA -- and which of
    its two softmax groups -- handles a tile's even and odd key blocks changes from run to run.  The output must not:
    three runs on the same inputs are bit-identical (a greedy decoder downstream turns a last-bit difference into
    another token at a near-tie)."""
    import ctypes as C
    B, H, S = 16, 16, 640
    n = B * H * S * 128
    q, k, v = (dev.empty(n, N.NS_BF16) for _ in range(3))
    for t, seed in ((q, 11), (k, 12), (v, 13)):
        N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_BF16, C.c_int64(n), seed, C.c_float(0.0), C.c_float(1.0))
    st = (C.c_int64 * 3)(H * S * 128, S * 128, 128)
    outs = []
    for rep in range(3):
        o = dev.zeros(n, N.NS_BF16)
        N.call("ns_attention_prefill", dev.handle, q.ptr, k.ptr, v.ptr, o.ptr, B, H, S, 128, st, st, st, st, C.c_float(0.0884), 1)
        dev.synchronize()
        outs.append(o.download())
        o.release()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
