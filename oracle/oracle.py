"""ctypes binding of the CPU oracle (oracle/ns_oracle.c) plus numpy helpers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs
of ``bench.py``; never by the ``nn_b200`` package.  Every function is a thin wrapper of the C function
of the same name, which cites the reference source it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libns_oracle.so")


def build(force: bool = False) -> str:
    """Compile libns_oracle.so with the Makefile beside this file (gcc only, a second or two)."""
    src = os.path.join(_HERE, "ns_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libns_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_counter_uniform.restype = C.c_float
        _lib.orc_counter_uniform.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        _lib.orc_get_threads.restype = C.c_int
        _lib.orc_gather.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(n))


def get_threads() -> int:
    return int(lib().orc_get_threads())


# ---------------------------------------------------------------- synthetic inputs
def normal(shape, seed: int, std: float = 1.0, mean: float = 0.0, offset: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    lib().orc_fill_normal(_p(out), C.c_int64(out.size), C.c_uint32(seed), C.c_uint64(offset), C.c_float(mean), C.c_float(std))
    return out


def token_ids(shape, seed: int, bound: int, offset: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    lib().orc_fill_ids(_p(out), C.c_int64(out.size), C.c_uint32(seed), C.c_uint64(offset), C.c_uint32(bound))
    return out


def counter_uniform(seed: int, step: int, row: int) -> float:
    return float(lib().orc_counter_uniform(seed, step, row))


# ---------------------------------------------------------------- float32 operators
def matmul_f32(a, b, batch, m, n, k, transA=False, transB=False, beta=0.0, c=None, scalar=False) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.zeros((batch, m, n), dtype=np.float32) if c is None else np.array(c, dtype=np.float32).reshape(batch, m, n)
    fn = lib().orc_matmul_f32_scalar if scalar else lib().orc_matmul_f32
    fn(_p(a), _p(b), _p(out), C.c_int(batch), C.c_int(m), C.c_int(n), C.c_int(k), C.c_int(int(transA)), C.c_int(int(transB)), C.c_float(beta))
    return out


def linear_f32(x, w_kn, bias=None) -> np.ndarray:
    """y = x . W + b with W [K,N] (Linear.ForwardCore, src/NeuralSharp/Layers/Linear.cs:43-47)."""
    x = _f32(x)
    k, n = w_kn.shape
    m = x.size // k
    y = matmul_f32(x, w_kn, 1, m, n, k).reshape(m, n)
    if bias is not None:
        y = add_rowvec(y, bias)
    return y.reshape(*x.shape[:-1], n)


def scale_mask_softmax(x, mask, scale: float) -> np.ndarray:
    x = _f32(x)
    cols = x.shape[-1]
    rows = x.size // cols
    y = np.empty_like(x)
    if mask is None:
        lib().orc_scale_mask_softmax(_p(x), None, _p(y), C.c_int(rows), C.c_int(cols), C.c_int(1), C.c_float(scale))
    else:
        mask = _f32(mask)
        lib().orc_scale_mask_softmax(_p(x), _p(mask), _p(y), C.c_int(rows), C.c_int(cols), C.c_int(mask.size // cols), C.c_float(scale))
    return y


def softmax(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_softmax(_p(x), _p(y), C.c_int(x.size // x.shape[-1]), C.c_int(x.shape[-1]))
    return y


def layernorm_fused(x, gamma, beta, eps: float = 1e-5) -> np.ndarray:
    x, gamma, beta = _f32(x), _f32(gamma), _f32(beta)
    y = np.empty_like(x)
    lib().orc_layernorm_fused(_p(x), _p(gamma), _p(beta), _p(y), C.c_int(x.size // x.shape[-1]), C.c_int(x.shape[-1]), C.c_float(eps))
    return y


def bias_gelu(x, bias) -> np.ndarray:
    x, bias = _f32(x), _f32(bias)
    y = np.empty_like(x)
    lib().orc_bias_gelu(_p(x), _p(bias), _p(y), C.c_int64(x.size), C.c_int(x.shape[-1]))
    return y


def add_rowvec(a, v) -> np.ndarray:
    a, v = _f32(a), _f32(v)
    c = np.empty_like(a)
    lib().orc_add_rowvec(_p(a), _p(v), _p(c), C.c_int64(a.size // a.shape[-1]), C.c_int(a.shape[-1]))
    return c


def decoder_mask(position: float, rows: int, capacity: int) -> np.ndarray:
    pos = np.array([position], dtype=np.float32)
    mask = np.empty((rows, capacity), dtype=np.float32)
    lib().orc_decoder_mask(_p(pos), _p(mask), C.c_int(rows), C.c_int(capacity))
    return mask


def kv_write(source, cache, position: float) -> None:
    """cache [heads, capacity, dim] is updated in place from source [heads, steps, dim]."""
    source = _f32(source)
    heads, steps, dim = source.shape
    assert cache.dtype == np.float32 and cache.shape[0] == heads and cache.shape[2] == dim
    pos = np.array([position], dtype=np.float32)
    lib().orc_kv_write(_p(source), _p(cache), _p(pos), C.c_int(heads), C.c_int(steps), C.c_int(cache.shape[1]), C.c_int(dim))


def gather(table, indices) -> np.ndarray:
    table, indices = _f32(table), _f32(indices)
    vocab, dim = table.shape
    y = np.empty((indices.size, dim), dtype=np.float32)
    rc = lib().orc_gather(_p(table), _p(indices), _p(y), C.c_int(indices.size), C.c_int(dim), C.c_int(vocab))
    if rc != 0:
        raise IndexError("embedding index is not an integer in [0, vocabulary)")
    return y.reshape(*indices.shape, dim)


def argmax(x) -> np.ndarray:
    x = _f32(x)
    rows = x.size // x.shape[-1]
    y = np.empty(rows, dtype=np.float32)
    lib().orc_argmax(_p(x), _p(y), C.c_int(rows), C.c_int(x.shape[-1]))
    return y


def sinusoid_table(max_length: int, dim: int) -> np.ndarray:
    t = np.empty((max_length, dim), dtype=np.float32)
    lib().orc_sinusoid_table(_p(t), C.c_int(max_length), C.c_int(dim))
    return t


# ---------------------------------------------------------------- bf16 / int8 rules
def round_bf16(x) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().orc_round_bf16(_p(x), _p(y), C.c_int64(x.size))
    return y


def widen_bf16(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    y = np.empty(h.shape, dtype=np.float32)
    lib().orc_widen_bf16(_p(h), _p(y), C.c_int64(h.size))
    return y


def bf16_round_trip(x) -> np.ndarray:
    return widen_bf16(round_bf16(x))


def quantize_rows_i8(x):
    """x [rows, cols] float32 (or uint16 bf16 bits) -> (int8 [rows, cols], float32 scale [rows])."""
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    if x.dtype == np.uint16:
        lib().orc_quantize_rows_i8_bf16(_p(x), C.c_int64(rows), C.c_int(cols), _p(q), _p(s))
    else:
        x = _f32(x)
        lib().orc_quantize_rows_i8(_p(x), C.c_int64(rows), C.c_int(cols), _p(q), _p(s))
    return q, s


def qmatmul_i8_acc(aq, wq, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    """Exact int32 accumulators of rows [row0, row0+nrows) of aq [M,K] against wq [N,K]."""
    aq = np.ascontiguousarray(aq, dtype=np.int8)
    wq = np.ascontiguousarray(wq, dtype=np.int8)
    M, K = aq.shape
    N = wq.shape[0]
    nrows = M - row0 if nrows is None else nrows
    acc = np.empty((nrows, N), dtype=np.int32)
    lib().orc_qmatmul_i8_acc(_p(aq), _p(wq), _p(acc), C.c_int(row0), C.c_int(nrows), C.c_int(N), C.c_int(K))
    return acc


def dequant_epilogue(acc, a_scale, w_scale, bias=None, residual=None, act: int = 0, row0: int = 0) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    nrows, N = acc.shape
    a_scale, w_scale = _f32(a_scale), _f32(w_scale)
    bias = None if bias is None else _f32(bias)
    residual = None if residual is None else _f32(residual)
    y = np.empty((nrows, N), dtype=np.float32)
    lib().orc_dequant_epilogue(_p(acc), _p(a_scale), _p(w_scale), None if bias is None else _p(bias),
                               None if residual is None else _p(residual), _p(y), C.c_int(row0), C.c_int(nrows), C.c_int(N), C.c_int(act))
    return y


def matmul_bf16(a_bits, b_bits, b_is_nk: bool, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    """float results of rows [row0,row0+nrows) of A [M,K] (bf16 bits) times B ([N,K] or [K,N], bf16 bits)."""
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    M, K = a_bits.shape
    N = b_bits.shape[0] if b_is_nk else b_bits.shape[1]
    nrows = M - row0 if nrows is None else nrows
    c = np.empty((nrows, N), dtype=np.float32)
    lib().orc_matmul_bf16(_p(a_bits), _p(b_bits), _p(c), C.c_int(row0), C.c_int(nrows), C.c_int(N), C.c_int(K), C.c_int(int(b_is_nk)))
    return c


def attention_slice(q, k, v, q_pos0: int, scale: float, causal: bool = True) -> np.ndarray:
    """One (batch, head) slice: q [tq, dh], k/v [tk, dh] float32 -> o [tq, dh] float32."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    tq, dh = q.shape
    tk = k.shape[0]
    o = np.empty((tq, dh), dtype=np.float32)
    lib().orc_attention_slice(_p(q), _p(k), _p(v), _p(o), C.c_int(tq), C.c_int(tk), C.c_int(dh),
                              C.c_int64(dh), C.c_int64(dh), C.c_int64(dh), C.c_int64(dh),
                              C.c_int(q_pos0), C.c_float(scale), C.c_int(int(causal)))
    return o


def close(expected, actual, tol: float) -> bool:
    """The reference's tolerance rule: |e - a| <= tol * max(1, |e|) (tests/NeuralSharp.Tests/Program.cs:572-583)."""
    e = np.asarray(expected, dtype=np.float64)
    a = np.asarray(actual, dtype=np.float64)
    return bool(np.all(np.abs(e - a) <= tol * np.maximum(1.0, np.abs(e))))


def max_err(expected, actual) -> float:
    """max |e - a| / max(1, |e|)."""
    e = np.asarray(expected, dtype=np.float64)
    a = np.asarray(actual, dtype=np.float64)
    return float(np.max(np.abs(e - a) / np.maximum(1.0, np.abs(e)))) if e.size else 0.0


# ---------------------------------------------------------------- token sampler
def sample_rows(logits, step: int, rows: int, vocabulary: int, row_stride: int, row_offset: int, temperature: float = 1.0,
                top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 0, stats=None):
    """Returns (ids [rows], stats [(step+1)*rows*13]) -- Backend.SampleRows (Backends/Backend.cs:248)."""
    logits = _f32(logits)
    ids = np.zeros(rows, dtype=np.float32)
    if stats is None:
        stats = np.zeros((step + 1) * rows * 13, dtype=np.float32)
    st = np.array([step], dtype=np.float32)
    lib().orc_sample_rows(_p(logits), _p(ids), _p(stats), _p(st), C.c_int(rows), C.c_int(vocabulary), C.c_int(row_stride), C.c_int(row_offset),
                          C.c_float(temperature), C.c_int(top_k), C.c_float(top_p), C.c_float(min_p), C.c_uint32(seed))
    return ids, stats


def penalize_rows(logits, history, length: int, rows: int, vocabulary: int, row_stride: int, row_offset: int, capacity: int, last_n: int,
                  repeat: float, presence: float, frequency: float) -> np.ndarray:
    logits, history = _f32(logits), _f32(history)
    work = np.zeros((rows, vocabulary), dtype=np.float32)
    ln = np.array([length], dtype=np.float32)
    lib().orc_penalize_rows(_p(logits), _p(work), _p(history), _p(ln), C.c_int(rows), C.c_int(vocabulary), C.c_int(row_stride), C.c_int(row_offset),
                            C.c_int(capacity), C.c_int(last_n), C.c_float(repeat), C.c_float(presence), C.c_float(frequency))
    return work


def history_push(ids, history, length: int, capacity: int) -> None:
    ids = _f32(ids)
    assert history.dtype == np.float32 and history.flags["C_CONTIGUOUS"]
    ln = np.array([length], dtype=np.float32)
    lib().orc_history_push(_p(ids), _p(history), _p(ln), C.c_int(ids.size), C.c_int(capacity))
