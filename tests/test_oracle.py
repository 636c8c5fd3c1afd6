"""The oracle against the reference's known answers and self-checking properties (no GPU).

Every case names the reference test it restates (tests/golden/kat.json holds the literals)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc

KAT = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "kat.json")))


def test_argmax_first_maximum_wins():
    k = KAT["argmax"]
    assert list(orc.argmax(np.array(k["x"], np.float32))) == k["expected"]
    assert list(orc.argmax(np.array([[1.0, 3.0, 3.0, 2.0]], np.float32))) == [1]


def test_softmax_stable_for_large_inputs():
    k = KAT["softmax_stable"]
    x = np.array([k["x"]], np.float32)
    assert orc.close(k["expected"], orc.softmax(x)[0], k["tol"])
    assert orc.close(k["expected"], orc.scale_mask_softmax(x, None, 1.0)[0], k["tol"])


def test_softmax_rows_against_double():
    x = orc.normal((4, 7), 30, 5.0)
    y = orc.softmax(x)
    for r in range(4):
        e = np.exp(x[r].astype(np.float64) - x[r].max())
        assert orc.close(e / e.sum(), y[r], 1e-5)


@pytest.mark.parametrize("m,n,k", KAT["matmul_shapes"]["shapes"])
def test_matmul_reference(m, n, k):
    """MatMulReference: all transposes and beta in {0,1} against double accumulation; the blocked AVX2 version
    (the timed CPU baseline) must be bit-identical to the scalar definition."""
    for ta in (False, True):
        for tb in (False, True):
            for beta in (0.0, 1.0):
                a = orc.normal((k, m) if ta else (m, k), 1 + m)
                b = orc.normal((n, k) if tb else (k, n), 2 + n)
                c0 = orc.normal((1, m, n), 3 + k)
                fast = orc.matmul_f32(a, b, 1, m, n, k, ta, tb, beta, c=c0)
                slow = orc.matmul_f32(a, b, 1, m, n, k, ta, tb, beta, c=c0, scalar=True)
                assert np.array_equal(fast.view(np.uint32), slow.view(np.uint32))
                A = (a.T if ta else a).astype(np.float64)
                B = (b.T if tb else b).astype(np.float64)
                assert orc.close(A @ B + beta * c0[0], fast[0], KAT["matmul_shapes"]["tol"])


def test_batched_matmul_and_thread_budget():
    k = KAT["batched_matmul"]
    a = orc.normal((k["batch"], k["m"], k["k"]), 31)
    b = orc.normal((k["batch"], k["k"], k["n"]), 32)
    got = orc.matmul_f32(a, b, k["batch"], k["m"], k["n"], k["k"])
    assert orc.close(a.astype(np.float64) @ b.astype(np.float64), got, k["tol"])
    # ThreadBudget (Program.cs:294-313): 300x200 . 200x100 identical with 1 and N threads
    a, b = orc.normal((300, 200), 33), orc.normal((200, 100), 34)
    n_threads = orc.get_threads()
    orc.set_threads(1)
    one = orc.matmul_f32(a, b, 1, 300, 100, 200)
    orc.set_threads(n_threads)
    many = orc.matmul_f32(a, b, 1, 300, 100, 200)
    assert np.array_equal(one, many)


def test_large_tensors():
    n = KAT["large_tensors"]["n"]
    a = orc.normal((n, n), 9)
    got = orc.matmul_f32(a, np.ones((n, 1), np.float32), 1, n, 1, n)
    assert orc.close(a.astype(np.float64).sum(axis=1), got[0, :, 0], KAT["large_tensors"]["tol"])


def test_fused_kernels_equal_unfused():
    k = KAT["fused_kernels"]
    x = orc.normal((6, 37), 41, 3.0)
    mask = np.where(np.arange(37)[None, :] <= np.arange(3)[:, None] + 20, 0.0, -1e9).astype(np.float32)
    fused = orc.scale_mask_softmax(x, mask, k["softmax_scale"])
    unfused = orc.softmax(x * np.float32(k["softmax_scale"]) + np.tile(mask, (2, 1)))
    assert orc.close(unfused, fused, k["softmax_tol"])
    # fused LayerNorm against the three-step definition in double
    g, b = orc.normal((37,), 42), orc.normal((37,), 43)
    xd = x.astype(np.float64)
    ln = (xd - xd.mean(1, keepdims=True)) / np.sqrt(xd.var(1, keepdims=True) + 1e-5) * g + b
    assert orc.close(ln, orc.layernorm_fused(x, g, b), k["layernorm_tol"])
    # bias + GELU == (x + b).Gelu()
    v = (x + g).astype(np.float64)
    gelu = 0.5 * v * (1 + np.tanh(0.7978845608 * (v + 0.044715 * v ** 3)))
    assert orc.close(gelu, orc.bias_gelu(x, g), k["bias_gelu_tol"])


def test_sampler_probabilities_and_counter_random():
    k = KAT["sampler_logits"]
    p = orc.softmax(np.array([k["logits"]], np.float32))[0]
    assert orc.close(k["probabilities"], p, k["tol"])
    assert list(np.argsort(-p)[:3]) == k["top_order"]
    # CounterRandom.Uniform restated independently in Python integers
    def ref(seed, step, row):
        h = (seed ^ (step * 0x9E3779B9) ^ (row * 0x85EBCA6B)) & 0xFFFFFFFF
        h ^= h >> 16; h = (h * 0x85EBCA6B) & 0xFFFFFFFF; h ^= h >> 13; h = (h * 0xC2B2AE35) & 0xFFFFFFFF; h ^= h >> 16
        return np.float32(h >> 8) * np.float32(1.0 / 16777216.0)
    for seed, step, row in [(0, 0, 0), (1, 2, 3), (12345, 77, 9), (0xFFFFFFFF, 1000, 63)]:
        u = orc.counter_uniform(seed, step, row)
        assert u == ref(seed, step, row) and 0.0 <= u < 1.0


def test_decoder_mask_kv_write_gather():
    m = orc.decoder_mask(4.0, 3, 12)
    assert m[0, 4] == 0 and m[0, 5] == np.float32(-1e9) and m[2, 6] == 0 and m[2, 7] == np.float32(-1e9)
    cache = np.zeros((2, 6, 3), np.float32)
    src = orc.normal((2, 2, 3), 5)
    orc.kv_write(src, cache, 3.0)
    assert np.array_equal(cache[:, 3:5], src) and not cache[:, :3].any() and not cache[:, 5:].any()
    table = orc.normal((5, 4), 6)
    assert np.array_equal(orc.gather(table, np.array([4, 0, 4], np.float32)), table[[4, 0, 4]])
    with pytest.raises(IndexError):   # the CPU backend throws on a non-integer or out-of-range id
        orc.gather(table, np.array([5.0], np.float32))
    with pytest.raises(IndexError):
        orc.gather(table, np.array([1.5], np.float32))


def test_causal_masking_property():
    """CausalMasking (AdvancedTests.cs:375-392): changing the last position leaves earlier outputs unchanged."""
    t, dh = 9, 8
    q, k, v = orc.normal((t, dh), 1), orc.normal((t, dh), 2), orc.normal((t, dh), 3)
    o1 = orc.attention_slice(q, k, v, 0, 1.0 / np.sqrt(dh))
    k2, v2, q2 = k.copy(), v.copy(), q.copy()
    k2[-1] += 1.0; v2[-1] -= 2.0; q2[-1] *= 3.0
    o2 = orc.attention_slice(q2, k2, v2, 0, 1.0 / np.sqrt(dh))
    assert orc.close(o1[:-1], o2[:-1], 1e-5) and not orc.close(o1[-1:], o2[-1:], 1e-5)


def test_cached_attention_equals_full():
    """CachedDecodingMatchesFull (DecodingTests.cs:69-98) at the attention level: a prefill of 4 positions and 6
    single steps over a zero-initialised cache of capacity 12 equal the full causal attention (1e-4)."""
    t, cap, dh = 10, 12, 8
    q, k, v = orc.normal((t, dh), 11), orc.normal((t, dh), 12), orc.normal((t, dh), 13)
    scale = 1.0 / np.sqrt(dh)
    full = orc.attention_slice(q, k, v, 0, scale)
    kc, vc = np.zeros((1, cap, dh), np.float32), np.zeros((1, cap, dh), np.float32)
    outs, pos = [], 0
    for steps in [4] + [1] * 6:
        orc.kv_write(k[None, pos:pos + steps], kc, float(pos))
        orc.kv_write(v[None, pos:pos + steps], vc, float(pos))
        outs.append(orc.attention_slice(q[pos:pos + steps], kc[0], vc[0], pos, scale))
        pos += steps
    assert orc.close(full, np.concatenate(outs), 1e-4)


def test_quantisation_rules():
    x = np.array([[0.0, 0.0, 0.0, 0.0], [1.0, -2.0, 0.5, 127.0], [2.5, 3.5, -2.5, 5.0]], np.float32)
    q, s = orc.quantize_rows_i8(x)
    assert s[0] == 1.0 and not q[0].any()                      # zero row: scale 1
    assert s[1] == 1.0 and list(q[1]) == [1, -2, 0, 127]        # 0.5 rounds to even (0)
    x2 = np.array([[0.5, 1.5, 2.5, -3.5, 127.0]], np.float32)
    q2, s2 = orc.quantize_rows_i8(x2)
    assert s2[0] == 1.0 and list(q2[0]) == [0, 2, 2, -4, 127]   # round half to even
    assert q.min() >= -127 and q.max() <= 127
    # bf16 rounding: nearest even on the 16th bit
    b = orc.round_bf16(np.array([1.0, 1.00390625, 1.01171875, -3.0e38], np.float32))
    assert list(orc.widen_bf16(b)[:3]) == [1.0, 1.0, 1.015625]
    # exact int32 accumulation and the order of the dequantising epilogue
    aq = np.array([[127, -127, 5, 0]], np.int8)
    wq = np.array([[127, 127, 1, 9], [-127, 127, 2, 9]], np.int8)
    acc = orc.qmatmul_i8_acc(aq, wq)
    assert list(acc[0]) == [5, -127 * 127 * 2 + 10]
    a_s, w_s, bias = np.array([0.1], np.float32), np.array([0.3, 0.7], np.float32), np.array([1.0, -1.0], np.float32)
    y = orc.dequant_epilogue(acc, a_s, w_s, bias)
    exp = (np.float32(acc[0].astype(np.float32) * a_s[0]) * w_s) + bias
    assert np.array_equal(y[0], exp.astype(np.float32))


def test_sinusoid_table():
    t = orc.sinusoid_table(6, 8)
    assert t[0, 0] == 0.0 and t[0, 1] == 1.0
    assert abs(t[3, 2] - np.sin(3 / 10000 ** (2 / 8))) < 1e-6 and abs(t[3, 3] - np.cos(3 / 10000 ** (2 / 8))) < 1e-6
