"""bf16 x bf16 -> float product (ns_matmul_bf16) against the oracle: <= 1e-2 relative, |e-a| <= tol*max(1,|e|).

Config: squares {1024, 4096, 8192} and the skinny shape M=8, K=4096, N=14336 (benchmark configuration "bf16 dense MatMul",
seed 2); B is stored [K, N] as in the config (and as Linear.Weight in the reference) and also [N, K].
"""
import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run(dev, a_bits, b_bits, m, n, k, transB, out_dtype=N.NS_BF16, batch=1, bias=None, epilogue=N.EPI_NONE):
    d_a, d_b = dev.from_numpy(a_bits), dev.from_numpy(b_bits)
    d_c = dev.empty(batch * m * n, out_dtype)
    d_bias = dev.from_numpy(bias) if bias is not None else None
    N.call("ns_matmul_bf16", dev.handle, d_a.ptr, d_b.ptr, d_c.ptr, batch, m, n, k, int(transB), d_bias.ptr if d_bias else 0, 0, 0,
           epilogue, out_dtype)
    dev.synchronize()
    return d_c.download((batch, m, n))


@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (3, 16, 24), (17, 40, 72), (64, 48, 72), (130, 72, 96), (128, 256, 64), (257, 520, 1032)])
def test_small_shapes(dev, orc, m, n, k, transB):
    a = orc.round_bf16(orc.normal((m, k), 21))
    b = orc.round_bf16(orc.normal((n, k) if transB else (k, n), 22))
    c = _run(dev, a, b, m, n, k, transB, out_dtype=N.NS_F32)[0]
    exp = orc.matmul_bf16(a, b, b_is_nk=transB)
    assert orc.close(exp, c, 1e-4), f"max err {orc.max_err(exp, c)}"   # float output of a short sum: accumulation-order noise only
    cb = _run(dev, a, b, m, n, k, transB, out_dtype=N.NS_BF16)[0]
    assert orc.close(orc.widen_bf16(orc.round_bf16(exp)), orc.widen_bf16(cb), TOL)


def test_batched_and_bias(dev, orc):
    batch, m, n, k = 3, 40, 64, 128
    a = orc.round_bf16(orc.normal((batch, m, k), 23))
    b = orc.round_bf16(orc.normal((batch, k, n), 24))
    bias = orc.normal((n,), 25)
    c = _run(dev, a, b, m, n, k, False, out_dtype=N.NS_F32, batch=batch, bias=bias, epilogue=N.EPI_BIAS)
    for i in range(batch):
        exp = orc.matmul_bf16(a[i], b[i], b_is_nk=False) + bias[None, :]
        assert orc.close(exp, c[i], 1e-4)


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192), (8, 14336, 4096)])
def test_baseline_shapes(dev, orc, m, n, k):
    """Oracle on sampled rows; B stored [K, N] as the config states."""
    a = orc.round_bf16(orc.normal((m, k), 2))
    b = orc.round_bf16(orc.normal((k, n), 3))
    c = _run(dev, a, b, m, n, k, False, out_dtype=N.NS_BF16)[0]
    rows = sorted(set([0, m - 1, m // 2] + list(np.random.default_rng(7).integers(0, m, 5))))
    bt = np.ascontiguousarray(b.T)  # [N, K] for the oracle's inner loop
    for r in rows:
        exp = orc.matmul_bf16(a[r:r + 1], bt, b_is_nk=True)
        assert orc.close(orc.widen_bf16(orc.round_bf16(exp)), orc.widen_bf16(c[r:r + 1]), TOL), f"row {r}: {orc.max_err(exp, orc.widen_bf16(c[r:r+1]))}"
    # linearity property on the full output: (column sums of C) ~= (column sums of A) . B, in float64
    if m <= 4096:
        a_sum = orc.widen_bf16(a).astype(np.float64).sum(axis=0)
        exp_cols = a_sum @ orc.widen_bf16(b).astype(np.float64)
        got_cols = orc.widen_bf16(c).astype(np.float64).sum(axis=0)
        # each output is rounded to bf16 (relative error <= 2^-9), so a column sum is off by at most 2^-9 * sum |c|;
        # the float accumulation adds far less.  Bound used: 2^-8 * sum |c| + 1e-3.
        bound = 2.0 ** -8 * np.abs(orc.widen_bf16(c).astype(np.float64)).sum(axis=0) + 1e-3
        assert np.all(np.abs(exp_cols - got_cols) <= bound)


@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (257, 520, 1032), (900, 264, 512)])
def test_cta_pair_kernel(dev, orc, m, n, k, transB):
    """The two-CTA kernel forced onto small shapes, B stored [N, K] and [K, N]."""
    a = orc.round_bf16(orc.normal((m, k), 31))
    b = orc.round_bf16(orc.normal((n, k) if transB else (k, n), 32))
    dev.tune(512, 1)
    try:
        c = _run(dev, a, b, m, n, k, transB, out_dtype=N.NS_F32)[0]
    finally:
        dev.tune(0, 0)
    exp = orc.matmul_bf16(a, b, b_is_nk=transB)
    assert orc.close(exp, c, 1e-4), f"max err {orc.max_err(exp, c)}"


def test_equals_the_reference_float_product_on_widened_operands(dev, orc):
    """The reference's float product (CpuMatMul.cs:102-148, one FMA chain over k per output) on the bf16 operands widened
    to float is the same sum in another order: float output within K * 2^-23 of the terms' magnitudes."""
    m, n, k = 96, 384, 2048
    a = orc.round_bf16(orc.normal((m, k), 41))
    b = orc.round_bf16(orc.normal((k, n), 42))
    c = _run(dev, a, b, m, n, k, False, out_dtype=N.NS_F32)[0]
    af, bf = orc.widen_bf16(a), orc.widen_bf16(b)
    ref = orc.matmul_f32(af, bf, 1, m, n, k)
    bound = k * 2.0 ** -23 * (np.abs(af).astype(np.float64) @ np.abs(bf).astype(np.float64))
    assert np.all(np.abs(ref.astype(np.float64) - c.astype(np.float64)) <= bound)


def test_chained_products_without_synchronisation(dev, orc):
    """C1 = A . B then C2 = D . C1 queued back to back: the second product's B operand is what the first one writes.  A
    product may begin while the kernel before it is still running (programmatic dependent launch), so the raw entry
    point must not fetch B before that kernel has finished; the early fetch is reserved for Linear objects."""
    m, k, n, m2 = 256, 512, 384, 192
    a = orc.round_bf16(orc.normal((m, k), 51))
    b = orc.round_bf16(orc.normal((k, n), 52, 0.05))
    dmat = orc.round_bf16(orc.normal((m2, m), 53, 0.05))
    d_a, d_b, d_d = dev.from_numpy(a), dev.from_numpy(b), dev.from_numpy(dmat)
    for rep in range(3):
        c1 = dev.zeros(m * n, N.NS_BF16)
        c2 = dev.empty(m2 * n, N.NS_F32)
        dev.synchronize()
        N.call("ns_matmul_bf16", dev.handle, d_a.ptr, d_b.ptr, c1.ptr, 1, m, n, k, 0, 0, 0, 0, N.EPI_NONE, N.NS_BF16)
        N.call("ns_matmul_bf16", dev.handle, d_d.ptr, c1.ptr, c2.ptr, 1, m2, n, m, 0, 0, 0, 0, N.EPI_NONE, N.NS_F32)
        dev.synchronize()
        c1_host = c1.download((m, n))
        exp = orc.matmul_bf16(dmat, c1_host, b_is_nk=False)
        assert orc.close(exp, c2.download((m2, n)), 1e-4), f"repetition {rep}: the second product read B before it was written"


@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("m,n,k", [(700, 264, 512), (1024, 768, 1024)])
def test_cta_pair_kernel_with_k_blocks_dealt_out_evenly(dev, orc, m, n, k, transB):
    """The pair kernel with the tiles' k-blocks dealt out in equal shares (see the int8 test of the same name): float
    accumulators of a shared tile are added in a fixed order, so two runs agree bit for bit and with the oracle to 1e-4."""
    a = orc.round_bf16(orc.normal((m, k), 33))
    b = orc.round_bf16(orc.normal((n, k) if transB else (k, n), 34))
    dev.tune(512, 2)
    try:
        c1 = _run(dev, a, b, m, n, k, transB, out_dtype=N.NS_F32)[0]
        c2 = _run(dev, a, b, m, n, k, transB, out_dtype=N.NS_F32)[0]
    finally:
        dev.tune(0, 0)
    exp = orc.matmul_bf16(a, b, b_is_nk=transB)
    assert orc.close(exp, c1, 1e-4), f"max err {orc.max_err(exp, c1)}"
    assert np.array_equal(c1.view(np.uint32), c2.view(np.uint32))
