"""int8 x int8 -> int32 product with the dequantising epilogue (ns_qmatmul_i8) against the oracle.

Accumulators must be bit-exact; the float epilogue is computed in the same operation order as the oracle, so
it is compared bit-exactly too (tolerance 0) except through GELU, where tanhf differs by ulps (1e-5).
Config: K = N = 4096, M in {1, 16, 128, 2048, 8192} (benchmark configuration "int8 QuantizedMatMul sweep", seed 1).
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N

pytestmark = pytest.mark.gpu


def _run(dev, aq, a_scale, wq, w_scale, bias=None, residual=None, epilogue=N.EPI_NONE, out_dtype=N.NS_F32, want_raw=True,
         residual_dtype=N.NS_F32):
    M, K = aq.shape
    Nn = wq.shape[0]
    d_a, d_w = dev.from_numpy(aq), dev.from_numpy(wq)
    d_as, d_ws = dev.from_numpy(a_scale), dev.from_numpy(w_scale)
    d_b = dev.from_numpy(bias) if bias is not None else None
    d_r = dev.from_numpy(residual) if residual is not None else None
    d_y = dev.empty(M * Nn, out_dtype)
    d_raw = dev.empty(M * Nn, N.NS_I32) if want_raw else None
    N.call("ns_qmatmul_i8", dev.handle, d_a.ptr, d_as.ptr, d_w.ptr, d_ws.ptr, d_b.ptr if d_b else 0, d_r.ptr if d_r else 0,
           residual_dtype, M, Nn, K, epilogue, out_dtype, d_y.ptr, d_raw.ptr if d_raw else 0)
    dev.synchronize()
    y = d_y.download((M, Nn))
    raw = d_raw.download((M, Nn)) if want_raw else None
    return y, raw


def _inputs(orc, M, Nn, K, seed=1):
    a = orc.normal((M, K), seed, 1.0)
    w = orc.normal((Nn, K), seed + 100, 0.02)
    bias = orc.normal((Nn,), seed + 200, 0.01)
    aq, a_s = orc.quantize_rows_i8(a)
    wq, w_s = orc.quantize_rows_i8(w)
    return aq, a_s, wq, w_s, bias


@pytest.mark.parametrize("M,Nn,K", [(1, 64, 16), (3, 40, 48), (17, 33 * 4, 144), (128, 256, 128), (130, 72, 1040),
                                    (129, 520, 4096), (64, 2048, 8192), (300, 1000, 256)])
def test_small_shapes_bit_exact(dev, orc, M, Nn, K):
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=11)
    y, raw = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
    acc = orc.qmatmul_i8_acc(aq, wq)
    assert np.array_equal(raw, acc), f"accumulators differ at {np.argwhere(raw != acc)[:4]}"
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias)
    assert np.array_equal(y.view(np.uint32), exp.view(np.uint32)), f"max err {orc.max_err(exp, y)}"


@pytest.mark.parametrize("tile_n,splits", [(64, 1), (128, 1), (256, 1), (64, 4), (128, 3), (256, 2)])
def test_tilings_and_split_k(dev, orc, tile_n, splits):
    M, Nn, K = 200, 768, 2048
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=12)
    dev.tune(tile_n, splits)
    try:
        y, raw = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
    finally:
        dev.tune(0, 0)
    acc = orc.qmatmul_i8_acc(aq, wq)
    assert np.array_equal(raw, acc)
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias)
    assert np.array_equal(y.view(np.uint32), exp.view(np.uint32))


def test_epilogues(dev, orc):
    M, Nn, K = 96, 512, 512
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=13)
    acc = orc.qmatmul_i8_acc(aq, wq)
    res = orc.normal((M, Nn), 77, 1.0)
    # none
    y, _ = _run(dev, aq, a_s, wq, w_s, None, epilogue=N.EPI_NONE)
    assert np.array_equal(y.view(np.uint32), orc.dequant_epilogue(acc, a_s, w_s).view(np.uint32))
    # bias + gelu (tanhf differs by ulps between libm and CUDA)
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS_GELU)
    assert orc.close(orc.dequant_epilogue(acc, a_s, w_s, bias, act=1), y, 1e-5)
    # bias + residual (float residual)
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=N.EPI_BIAS_RESIDUAL)
    assert np.array_equal(y.view(np.uint32), orc.dequant_epilogue(acc, a_s, w_s, bias, residual=res).view(np.uint32))
    # bf16 residual and bf16 output
    res_b = orc.round_bf16(res)
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res_b, epilogue=N.EPI_BIAS_RESIDUAL, out_dtype=N.NS_BF16, residual_dtype=N.NS_BF16)
    exp = orc.round_bf16(orc.dequant_epilogue(acc, a_s, w_s, bias, residual=orc.widen_bf16(res_b)))
    assert np.array_equal(y, exp)


@pytest.mark.parametrize("M", [1, 16, 128, 2048, 8192])
def test_baseline_sweep(dev, orc, M):
    """K = N = 4096.  Oracle on sampled rows (all rows when M <= 128); exact row/column checksums on everything."""
    K = Nn = 4096
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=1)
    y, raw = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
    rows = list(range(M)) if M <= 128 else sorted(set([0, 1, 127, 128, 129, M // 2, M - 129, M - 2, M - 1] +
                                                      list(np.random.default_rng(5).integers(0, M, 24))))
    for r in rows:
        acc = orc.qmatmul_i8_acc(aq, wq, r, 1)
        assert np.array_equal(raw[r:r + 1], acc), f"row {r}"
        exp = orc.dequant_epilogue(acc, a_s, w_s, bias, row0=r)
        assert np.array_equal(y[r:r + 1].view(np.uint32), exp.view(np.uint32)), f"row {r}"
    # size-independent property: sum_n acc[m, n] == aq[m, :] . sum_n wq[n, :]  and  sum_m acc[m, n] == (sum_m aq[m, :]) . wq[n, :]
    wsum = wq.astype(np.int64).sum(axis=0)
    asum = aq.astype(np.int64).sum(axis=0)
    assert np.array_equal(raw.astype(np.int64).sum(axis=1), aq.astype(np.int64) @ wsum)
    assert np.array_equal(raw.astype(np.int64).sum(axis=0), wq.astype(np.int64) @ asum)


def test_extreme_values(dev, orc):
    """All operands at +-127: the largest accumulator magnitude K * 127^2 must be exact."""
    M, Nn, K = 128, 64, 8192
    aq = np.full((M, K), 127, np.int8)
    aq[1::2] = -127
    wq = np.full((Nn, K), -127, np.int8)
    ones_m, ones_n = np.ones(M, np.float32), np.ones(Nn, np.float32)
    _, raw = _run(dev, aq, ones_m, wq, ones_n)
    assert np.array_equal(raw, orc.qmatmul_i8_acc(aq, wq))
    assert raw.min() == -K * 127 * 127 and raw.max() == K * 127 * 127


def test_argument_errors(dev):
    with pytest.raises(N.NsError):
        N.call("ns_qmatmul_i8", dev.handle, 0, 0, 0, 0, 0, 0, 0, 4, 4, 16, 0, 0, 0, 0)
    a = dev.empty(64, N.NS_I8)
    s = dev.empty(64, N.NS_F32)
    with pytest.raises(N.NsError):  # K not a multiple of 16
        N.call("ns_qmatmul_i8", dev.handle, a.ptr, s.ptr, a.ptr, s.ptr, 0, 0, 0, 2, 2, 24, 0, 0, s.ptr, 0)
    with pytest.raises(N.NsError):  # bias epilogue without a bias
        N.call("ns_qmatmul_i8", dev.handle, a.ptr, s.ptr, a.ptr, s.ptr, 0, 0, 0, 2, 2, 16, N.EPI_BIAS, 0, s.ptr, 0)


@pytest.mark.parametrize("M,Nn,K", [(256, 256, 128), (129, 520, 4096), (300, 1000, 256), (700, 264, 1040), (1024, 768, 2048)])
@pytest.mark.parametrize("epi", [N.EPI_BIAS, N.EPI_BIAS_RESIDUAL])
def test_cta_pair_kernel_bit_exact(dev, orc, M, Nn, K, epi):
    """The two-CTA kernel (256 x 256 tiles, tcgen05 cta_group::2), forced onto shapes small enough for the oracle:
    full tiles, ragged rows (second CTA partly or wholly past M), ragged columns, many k-blocks (the 6-stage ring
    wraps), several tiles per cluster (both accumulators in use)."""
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=13)
    res = orc.normal((M, Nn), 77) if epi == N.EPI_BIAS_RESIDUAL else None
    dev.tune(512, 1)
    try:
        y, raw = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=epi)
        yb, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=epi, out_dtype=N.NS_BF16, want_raw=False)
    finally:
        dev.tune(0, 0)
    acc = orc.qmatmul_i8_acc(aq, wq)
    assert np.array_equal(raw, acc), f"accumulators differ at {np.argwhere(raw != acc)[:4]}"
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias, residual=res)
    assert np.array_equal(y.view(np.uint32), exp.view(np.uint32)), f"max err {orc.max_err(exp, y)}"
    assert np.array_equal(yb, orc.round_bf16(exp))


@pytest.mark.parametrize("M,Nn,K", [(1, 4096, 4096), (1, 37, 16), (2, 130, 528), (3, 1000, 1040), (4, 512, 16384), (5, 96, 2048),
                                    (8, 2048, 8192), (9, 333, 4096), (16, 1024, 8192), (16, 6, 512), (8, 6, 512), (7, 10, 16), (13, 4096, 2048), (2, 256, 32768),
                                    (1, 64, 32768), (1, 72, 16384), (4, 64, 32768), (8, 40, 16384), (2, 64, 16400)])
def test_row_streaming_kernel_bit_exact(dev, orc, M, Nn, K):
    """One to eight rows take the row-streaming kernel on the CUDA cores (every register shape: 1/2/4/8 rows x 1/2/4
    pieces per warp; ragged K pieces, ragged column groups, fewer columns than CTAs, one piece for a CTA whose
    epilogue needs two warps); nine to sixteen rows stay on the tensor cores.  Accumulators and every epilogue must
    equal the oracle's, and the tensor-core kernels' (forced by a tuning override) bit for bit."""
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=21)
    res = orc.normal((M, Nn), 78)
    acc = orc.qmatmul_i8_acc(aq, wq)
    y, raw = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
    assert np.array_equal(raw, acc), f"accumulators differ at {np.argwhere(raw != acc)[:4]}"
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias)
    assert np.array_equal(y.view(np.uint32), exp.view(np.uint32))
    y, _ = _run(dev, aq, a_s, wq, w_s, None, epilogue=N.EPI_NONE, want_raw=False)
    assert np.array_equal(y.view(np.uint32), orc.dequant_epilogue(acc, a_s, w_s).view(np.uint32))
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=N.EPI_BIAS_RESIDUAL, want_raw=False)
    exp_r = orc.dequant_epilogue(acc, a_s, w_s, bias, residual=res)
    assert np.array_equal(y.view(np.uint32), exp_r.view(np.uint32))
    res_b = orc.round_bf16(res)
    yb, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res_b, epilogue=N.EPI_BIAS_RESIDUAL, out_dtype=N.NS_BF16, residual_dtype=N.NS_BF16,
                 want_raw=False)
    assert np.array_equal(yb, orc.round_bf16(orc.dequant_epilogue(acc, a_s, w_s, bias, residual=orc.widen_bf16(res_b))))
    yg, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS_GELU, want_raw=False)
    assert orc.close(orc.dequant_epilogue(acc, a_s, w_s, bias, act=1), yg, 1e-5)
    # the tensor-core path on the same operands
    dev.tune(64, 2 if K >= 512 else 1)
    try:
        y_tc, raw_tc = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
        yg_tc, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS_GELU, want_raw=False)
    finally:
        dev.tune(0, 0)
    assert np.array_equal(raw_tc, acc)
    assert np.array_equal(y_tc.view(np.uint32), exp.view(np.uint32))
    assert np.array_equal(yg_tc.view(np.uint32), yg.view(np.uint32)), "GELU epilogue differs between the two kernels"


@pytest.mark.parametrize("M", [16, 128])
def test_equals_the_reference_float_linear_on_dequantised_operands(dev, orc, M):
    """The float32-only reference computes this Linear as x . W + b with its float product on whatever the operands
    are (Layers/Linear.cs:43-47 -> CpuMatMul.cs:102-148).  Given the de-quantised operands (aq * a_scale, wq * w_scale)
    that product must agree with the int8 path up to float rounding: the int8 path is exact up to its three final
    roundings, the float FMA chain over k carries at most K * 2^-24 of the sum of the terms' magnitudes."""
    K = Nn = 4096
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=1)
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS, want_raw=False)
    a_deq = (aq.astype(np.float32) * a_s[:, None]).astype(np.float32)          # exact in float: |q| <= 127
    w_deq_kn = np.ascontiguousarray((wq.astype(np.float32) * w_s[:, None]).T)    # Linear.Weight layout [K, N]
    ref = orc.matmul_f32(a_deq, w_deq_kn, 1, M, Nn, K) + bias[None, :]
    magnitude = np.abs(a_deq).astype(np.float64) @ np.abs(w_deq_kn).astype(np.float64) + np.abs(bias)[None, :]
    bound = K * 2.0 ** -23 * magnitude
    err = np.abs(ref.astype(np.float64) - y.astype(np.float64))
    assert np.all(err <= bound), f"largest excess {float((err - bound).max()):.3e}"
    # that worst-case bound is loose (a few per cent of a typical output); the float-accumulation bar of the benchmark
    # configuration, 1e-4 with the reference's rule |e - a| <= tol * max(1, |e|), holds as well
    assert orc.close(ref[0], y, 1e-4), f"max err {orc.max_err(ref[0], y):.3e}"


@pytest.mark.parametrize("M,Nn,K", [(700, 264, 1040), (1024, 768, 2048), (257, 520, 4096), (900, 1000, 256)])
@pytest.mark.parametrize("epi", [N.EPI_BIAS, N.EPI_BIAS_RESIDUAL])
def test_cta_pair_kernel_with_k_blocks_dealt_out_evenly(dev, orc, M, Nn, K, epi):
    """When the last wave of 256 x 256 tiles would leave many clusters idle (2048 x 4096: 128 tiles on 74 clusters), the
    pair kernel deals the tiles' k-blocks out in equal shares, and a tile that straddles two clusters is completed
    through a work area (its last k-blocks are computed first by one cluster, its first k-blocks last by the other,
    which adds the two exact int32 parts).  Forced here on shapes the oracle can check in full: bit-exact accumulators
    and outputs, twice in a row (the arrival counts of the work area are cleared per launch)."""
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=17)
    res = orc.normal((M, Nn), 79) if epi == N.EPI_BIAS_RESIDUAL else None
    acc = orc.qmatmul_i8_acc(aq, wq)
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias, residual=res)
    dev.tune(512, 2)
    try:
        for rep in range(2):
            y, raw = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=epi)
            assert np.array_equal(raw, acc), f"repetition {rep}: accumulators differ at {np.argwhere(raw != acc)[:4]}"
            assert np.array_equal(y.view(np.uint32), exp.view(np.uint32)), f"repetition {rep}"
        yb, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=epi, out_dtype=N.NS_BF16, want_raw=False)
    finally:
        dev.tune(0, 0)
    assert np.array_equal(yb, orc.round_bf16(exp))


@pytest.mark.parametrize("M,Nn,K", [(9, 40, 64), (16, 4096, 4096), (16, 1001, 8192), (13, 132, 144), (12, 6, 1040), (16, 2048, 2048), (10, 520, 2048),
                                    (16, 777, 1024), (11, 64, 4096), (16, 6144, 2048), (16, 3, 16), (15, 1000, 1040), (16, 32000, 256)])
def test_streaming_kernel_for_9_to_16_rows_bit_exact(dev, orc, M, Nn, K):
    """Nine to sixteen rows take the one-launch streaming kernel (weights straight into registers, mma.sync.m16n8k32, K
    summed inside the CTA): every register shape (1, 2, 4, 8 K groups per warp), ragged K groups, columns that are no
    multiple of 8, fewer column tiles than CTAs.  Accumulators and every epilogue equal the oracle's and the tcgen05
    kernels' (forced by the tuning hook) bit for bit."""
    aq, a_s, wq, w_s, bias = _inputs(orc, M, Nn, K, seed=23)
    res = orc.normal((M, Nn), 80)
    acc = orc.qmatmul_i8_acc(aq, wq)
    y, raw = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
    assert np.array_equal(raw, acc), f"accumulators differ at {np.argwhere(raw != acc)[:4]}"
    exp = orc.dequant_epilogue(acc, a_s, w_s, bias)
    assert np.array_equal(y.view(np.uint32), exp.view(np.uint32))
    y, _ = _run(dev, aq, a_s, wq, w_s, None, epilogue=N.EPI_NONE, want_raw=False)
    assert np.array_equal(y.view(np.uint32), orc.dequant_epilogue(acc, a_s, w_s).view(np.uint32))
    res_b = orc.round_bf16(res)
    yb, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res_b, epilogue=N.EPI_BIAS_RESIDUAL, out_dtype=N.NS_BF16, residual_dtype=N.NS_BF16,
                 want_raw=False)
    assert np.array_equal(yb, orc.round_bf16(orc.dequant_epilogue(acc, a_s, w_s, bias, residual=orc.widen_bf16(res_b))))
    y, _ = _run(dev, aq, a_s, wq, w_s, bias, residual=res, epilogue=N.EPI_BIAS_RESIDUAL, want_raw=False)
    assert np.array_equal(y.view(np.uint32), orc.dequant_epilogue(acc, a_s, w_s, bias, residual=res).view(np.uint32))
    yg, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS_GELU, want_raw=False)
    assert orc.close(orc.dequant_epilogue(acc, a_s, w_s, bias, act=1), yg, 1e-5)
    dev.tune(64, 2 if K >= 512 else 1)
    try:
        y_tc, raw_tc = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS)
        yg_tc, _ = _run(dev, aq, a_s, wq, w_s, bias, epilogue=N.EPI_BIAS_GELU, want_raw=False)
    finally:
        dev.tune(0, 0)
    assert np.array_equal(raw_tc, acc)
    assert np.array_equal(y_tc.view(np.uint32), exp.view(np.uint32))
    assert np.array_equal(yg_tc.view(np.uint32), yg.view(np.uint32)), "GELU epilogue differs between the two kernels"
