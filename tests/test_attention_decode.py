"""Cached attention (ns_kv_append + ns_attention_decode) against the oracle's reference-order attention.

bf16 keys/values/queries, float math; tolerance 1e-2 relative on bf16 outputs (|e-a| <= tol*max(1,|e|)).
Covers the reference's CachedDecodingMatchesFull / BatchedDecoding pattern (DecodingTests.cs:69-142): a prefill
followed by single steps equals full causal attention; identity and shuffled page tables give the same answer;
benchmark configuration 4's decode case (batch 64, 32 heads, cache length 4096, head_dim 128) on sampled (batch, head) pairs.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu
TOL = 1e-2


class Cache:
    def __init__(self, dev, batch, heads, dh, capacity, page_size, shuffle_seed=None):
        self.dev, self.batch, self.heads, self.dh, self.page_size = dev, batch, heads, dh, page_size
        self.max_pages = (capacity + page_size - 1) // page_size
        n_pages = batch * self.max_pages
        table = np.arange(n_pages, dtype=np.int32)
        if shuffle_seed is not None:
            np.random.default_rng(shuffle_seed).shuffle(table)
        self.table_host = table.reshape(batch, self.max_pages)
        self.table = dev.from_numpy(self.table_host)
        h = C.c_void_p()
        N.call("ns_kv_cache_create", dev.handle, n_pages, page_size, heads, dh, C.byref(h))
        self.handle = h
        self.pos = dev.from_numpy(np.array([0], np.int32))

    def append(self, k_bits, v_bits, steps):
        """k_bits, v_bits: uint16 [batch, steps, heads*dh]"""
        dk, dv = self.dev.from_numpy(k_bits), self.dev.from_numpy(v_bits)
        N.call("ns_kv_append", self.dev.handle, self.handle, dk.ptr, dv.ptr, C.c_int64(self.heads * self.dh), self.table.ptr, self.max_pages,
               self.pos.ptr, self.batch, steps)
        self.dev.synchronize()

    def attend(self, q_bits, steps, scale):
        dq = self.dev.from_numpy(q_bits)
        do = self.dev.empty(q_bits.size, N.NS_BF16)
        D = self.heads * self.dh
        N.call("ns_attention_decode", self.dev.handle, self.handle, dq.ptr, C.c_int64(D), do.ptr, C.c_int64(D), self.table.ptr, self.max_pages,
               self.pos.ptr, self.batch, steps, C.c_float(scale))
        self.dev.synchronize()
        return do.download((self.batch, steps, self.heads, self.dh))

    def advance(self, steps):
        N.call("ns_add_i32", self.dev.handle, self.pos.ptr, steps)

    def close(self):
        N.call("ns_kv_cache_destroy", self.handle)


@pytest.mark.parametrize("dh,heads,page_size,shuffle", [(128, 2, 16, None), (128, 2, 16, 5), (64, 3, 8, 7), (32, 4, 4, None)])
def test_prefill_then_steps_equals_full(dev, orc, dh, heads, page_size, shuffle):
    B, T, cap = 3, 37, 48
    scale = 1.0 / np.sqrt(dh)
    q = orc.round_bf16(orc.normal((B, T, heads, dh), 1))
    k = orc.round_bf16(orc.normal((B, T, heads, dh), 2))
    v = orc.round_bf16(orc.normal((B, T, heads, dh), 3))
    cache = Cache(dev, B, heads, dh, cap, page_size, shuffle)
    outs, pos = [], 0
    for steps in [20] + [1] * 12 + [5]:
        sl = slice(pos, pos + steps)
        cache.append(k[:, sl].reshape(B, steps, -1), v[:, sl].reshape(B, steps, -1), steps)
        outs.append(cache.attend(q[:, sl].reshape(B, steps, -1), steps, scale))
        cache.advance(steps)
        pos += steps
    got = orc.widen_bf16(np.concatenate(outs, axis=1))
    qf, kf, vf = orc.widen_bf16(q), orc.widen_bf16(k), orc.widen_bf16(v)
    for b in range(B):
        for h in range(heads):
            exp = orc.attention_slice(qf[b, :, h], kf[b, :, h], vf[b, :, h], 0, scale)
            assert orc.close(orc.bf16_round_trip(exp), got[b, :, h], TOL), (b, h, orc.max_err(exp, got[b, :, h]))
    cache.close()


def test_split_along_the_cache(dev, orc):
    """Few (batch, head) rows and a long cache: the kernel splits the cache across CTAs and merges the parts."""
    B, heads, dh, L, page_size = 1, 2, 128, 3000, 64
    scale = 1.0 / np.sqrt(dh)
    k = orc.round_bf16(orc.normal((B, L, heads, dh), 11))
    v = orc.round_bf16(orc.normal((B, L, heads, dh), 12))
    q = orc.round_bf16(orc.normal((B, 1, heads, dh), 13, 3.0))
    cache = Cache(dev, B, heads, dh, 4096, page_size, shuffle_seed=3)
    cache.append(k.reshape(B, L, -1), v.reshape(B, L, -1), L)
    cache.advance(L - 1)   # the query sits at the last written position
    got = orc.widen_bf16(cache.attend(q.reshape(B, 1, -1), 1, scale))
    for h in range(heads):
        exp = orc.attention_slice(orc.widen_bf16(q[0, :, h]), orc.widen_bf16(k[0, :, h]), orc.widen_bf16(v[0, :, h]), L - 1, scale)
        assert orc.close(orc.bf16_round_trip(exp), got[0, :, h], TOL), orc.max_err(exp, got[0, :, h])
    cache.close()


def test_baseline_decode_shape(dev, orc):
    """batch 64, 32 heads, head_dim 128, cache length 4096 (+1 for the new token); pools filled on the device,
    oracle on sampled (batch, head) pairs read back from the pools."""
    B, heads, dh, L, page_size = 64, 32, 128, 4096, 64
    scale = 1.0 / np.sqrt(dh)
    cache = Cache(dev, B, heads, dh, L + page_size, page_size)
    kp, vp, nbytes = C.c_uint64(), C.c_uint64(), C.c_uint64()
    N.call("ns_kv_cache_pools", cache.handle, C.byref(kp), C.byref(vp), C.byref(nbytes))
    N.call("ns_fill_normal", dev.handle, kp.value, N.NS_BF16, C.c_int64(nbytes.value // 2), 31, C.c_float(0.0), C.c_float(1.0))
    N.call("ns_fill_normal", dev.handle, vp.value, N.NS_BF16, C.c_int64(nbytes.value // 2), 32, C.c_float(0.0), C.c_float(1.0))
    q = orc.round_bf16(orc.normal((B, 1, heads, dh), 33))
    N.call("ns_add_i32", dev.handle, cache.pos.ptr, L - 1)
    got = orc.widen_bf16(cache.attend(q.reshape(B, 1, -1), 1, scale))
    from nn_b200.device import Storage
    slab = page_size * dh
    for (b, h) in [(0, 0), (63, 31), (17, 5), (40, 22)]:
        rows_k, rows_v = [], []
        for pg in range(L // page_size):
            page = int(cache.table_host[b, pg])
            off = (page * heads + h) * slab
            for pool, rows in ((kp.value, rows_k), (vp.value, rows_v)):
                buf = np.empty(slab, np.uint16)
                N.call("ns_d2h", dev.handle, buf.ctypes.data_as(C.c_void_p), C.c_uint64(pool + off * 2), C.c_uint64(slab * 2))
                rows.append(buf.reshape(page_size, dh))
        kf, vf = orc.widen_bf16(np.concatenate(rows_k)), orc.widen_bf16(np.concatenate(rows_v))
        exp = orc.attention_slice(orc.widen_bf16(q[b, :, h]), kf, vf, L - 1, scale)
        assert orc.close(orc.bf16_round_trip(exp), got[b, :, h], TOL), (b, h, orc.max_err(exp, got[b, :, h]))
    cache.close()


def test_append_outside_the_cache_is_skipped_and_reported(dev, orc):
    """A page-table entry that names no page of the pool, or a position beyond the table: nothing is written, the next
    synchronisation reports NS_ERR_KERNEL (status 500), and the device stays usable.  (The reference throws for a
    position beyond the capacity: DecodingContext.BeginStep, Layers/Decoding.cs:96-99.)"""
    import ctypes as C
    B, heads, dh, page_size, max_pages = 2, 2, 64, 16, 4
    cache = C.c_void_p()
    N.call("ns_kv_cache_create", dev.handle, B * max_pages, page_size, heads, dh, C.byref(cache))
    kp, vp, nbytes = C.c_uint64(), C.c_uint64(), C.c_uint64()
    N.call("ns_kv_cache_pools", cache, C.byref(kp), C.byref(vp), C.byref(nbytes))
    k = dev.from_numpy(orc.round_bf16(orc.normal((B, heads * dh), 61)))
    v = dev.from_numpy(orc.round_bf16(orc.normal((B, heads * dh), 62)))

    def pool_bytes():
        host = np.empty(nbytes.value // 2, np.uint16)
        N.call("ns_d2h", dev.handle, host.ctypes.data_as(C.c_void_p), kp, nbytes)
        return host

    for table_host, pos0 in ((np.array([0, 1, 2, 3, 4, 5, 999, 7], np.int32), 35),      # sequence 1, page 2 -> entry 999
                             (np.arange(B * max_pages, dtype=np.int32), page_size * max_pages),   # position past the table
                             (np.arange(B * max_pages, dtype=np.int32), -3)):
        dev.synchronize()
        table = dev.from_numpy(table_host)
        pos = dev.from_numpy(np.array([pos0], np.int32))
        before = pool_bytes()
        N.call("ns_kv_append", dev.handle, cache, k.ptr, v.ptr, C.c_int64(heads * dh), table.ptr, max_pages, pos.ptr, B, 1)
        with pytest.raises(N.NsError) as err:
            dev.synchronize()
        assert err.value.code == 4 and "status 500" in str(err.value)
        after = pool_bytes()
        if pos0 == 35:
            # sequence 0 (a valid entry) was appended, sequence 1 was skipped
            changed = np.nonzero(before != after)[0]
            assert changed.size > 0 and changed.max() < 3 * heads * page_size * dh
        else:
            assert np.array_equal(before, after)
    # still usable
    table = dev.from_numpy(np.arange(B * max_pages, dtype=np.int32))
    pos = dev.from_numpy(np.array([5], np.int32))
    N.call("ns_kv_append", dev.handle, cache, k.ptr, v.ptr, C.c_int64(heads * dh), table.ptr, max_pages, pos.ptr, B, 1)
    dev.synchronize()
    N.call("ns_kv_cache_destroy", cache)


@pytest.mark.parametrize("cap,length", [(768, 1), (768, 383), (768, 384), (768, 385), (768, 700), (2048, 1500), (4096, 3000), (128, 100)])
def test_a_sequence_in_a_batch_equals_the_sequence_in_a_small_batch(dev, orc, cap, length):
    """The reference's BatchedDecoding property (DecodingTests.cs:100-142), bit for bit: with 64 sequences every (sequence,
    head) row is one CTA's; with 4 sequences the cache of a row is split over several CTAs and merged by a second kernel.  The
    kernels walk a row's cache in the same chunks (384 positions for a cache of 768, 1024 for 2048 or 4096) and fold the chunks'
    partial results in the same order with the same operations, so the output bits must not depend on the batch the sequence
    is decoded in."""
    heads, dh, page_size = 8, 128, 16
    scale = 1.0 / np.sqrt(dh)
    B = 64
    k = orc.round_bf16(orc.normal((B, length, heads, dh), 21))
    v = orc.round_bf16(orc.normal((B, length, heads, dh), 22))
    q = orc.round_bf16(orc.normal((B, 1, heads, dh), 23, 2.0))

    def run(rows):
        cache = Cache(dev, len(rows), heads, dh, cap, page_size, shuffle_seed=9)
        cache.append(k[rows].reshape(len(rows), length, -1), v[rows].reshape(len(rows), length, -1), length)
        cache.advance(length - 1)
        out = cache.attend(q[rows].reshape(len(rows), 1, -1), 1, scale)
        cache.close()
        return out

    big = run(list(range(B)))
    for rows in ([0, 1, 2, 3], [60, 61, 62, 63], [17]):
        small = run(rows)
        assert np.array_equal(small, big[rows]), f"sequences {rows} differ between a batch of {len(rows)} and a batch of {B}"
    exp = orc.attention_slice(orc.widen_bf16(q[5, :, 3]), orc.widen_bf16(k[5, :, 3]), orc.widen_bf16(v[5, :, 3]), length - 1, scale)
    assert orc.close(orc.bf16_round_trip(exp), orc.widen_bf16(big[5, :, 3]), TOL)
