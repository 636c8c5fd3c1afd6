"""Benchmark of the hot path: int8 QuantizedMatMul (int8 x int8 -> int32, per-channel dequant + bias epilogue).

Workload (benchmark configuration "int8 QuantizedMatMul sweep", the largest M): A [8192, 4096] float ~N(0,1) quantised per
row, W [4096, 4096] ~N(0,0.02) quantised per output channel, bias ~N(0,0.01), float output.  One step = one pass
of the product over one batch of 8192 rows.  With N > 1 GPUs every rank runs its own batch of rows against its own
copy of the weights (batch sharding, no data-path collective): weak scaling.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` is device-resident throughput, `e2e` is the same product through the C
ABI from pinned host buffers (float activations in, float result out, copies inside the timed region), `roofline`
compares the tcgen05 kernel with the tensor-core peak, `cpu_baseline` times the oracle's restatement of the
reference's CPU product on this host's cores.  `--impl reference` times that CPU restatement alone (the reference
is C#/.NET and cannot run here).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, NN = 8192, 4096, 4096
OPS = 2.0 * M * K * NN
ALGO_BYTES = NN * K + M * K + 4 * M * NN + 4 * (M + 2 * NN)
METRIC, UNIT = "int8_quantized_matmul_tops", "TOPS"
CONFIG = {"workload": "int8 QuantizedMatMul M=8192 K=4096 N=4096 (per-row A scales, per-channel W scales, bias, f32 out)",
          "l2": "4 operand/result sets rotated per step (704 MB footprint > 126 MB L2)", "seed": 1,
          "clocks_window": "nvidia-smi sampled every 200 ms over ~1 s of back-to-back steps that contains the timed region"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16": float(p["bf16_tflops"]), "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.path = gpu_index, None, f"/tmp/ns_b200_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.proc.wait()
        sm, smax, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8 or not f[0].isdigit() or int(f[0]) != self.gpu_index:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_tops(rows: int, reps: int):
    """The reference's CPU path for this Linear: float product on the de-quantised operands
    (Backends/Cpu/CpuMatMul.cs via the oracle's restatement), all host threads, `rows` rows of the batch."""
    from oracle import oracle as orc
    orc.set_threads(len(os.sched_getaffinity(0)))   # all host cores, whatever OMP_NUM_THREADS says
    a = orc.normal((rows, K), 1)
    w_kn = orc.normal((K, NN), 2, 0.02)   # Linear.Weight layout [K, N]
    orc.matmul_f32(a[:64], w_kn, 1, 64, NN, K)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.matmul_f32(a, w_kn, 1, rows, NN, K)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return 2.0 * rows * K * NN / best / 1e12, orc.get_threads(), best


def run_reference(args, rank):
    if rank != 0:
        return
    rows = 2048
    times = []
    from oracle import oracle as orc
    orc.set_threads(len(os.sched_getaffinity(0)))   # all host cores: the launcher of multi-rank runs sets OMP_NUM_THREADS=1
    a = orc.normal((rows, K), 1)
    w_kn = orc.normal((K, NN), 2, 0.02)
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        orc.matmul_f32(a, w_kn, 1, rows, NN, K)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    tops = 2.0 * rows * K * NN / (ms * 1e-3) / 1e12
    sample = f"{rows} of {M} rows per step, float32 on de-quantised operands, OpenMP over 4-row blocks"
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f32", "data": "synthetic", "config": CONFIG,
                      "cpu_baseline": {"value": tops, "unit": UNIT, "cores": orc.get_threads(), "kind": "port", "sample": sample},
                      "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_ours(args, rank, world, local_rank):
    from nn_b200 import native as N
    from nn_b200.device import Device

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = Device(local_rank)
    peaks = measured_peaks()

    # ---- operands resident in HBM: SETS rotating sets, generated and quantised on the device
    SETS = 4
    sets = []
    for s in range(SETS):
        x = dev.empty(M * K)
        w = dev.empty(NN * K)
        N.call("ns_fill_normal", dev.handle, x.ptr, N.NS_F32, C.c_int64(M * K), 1 + 16 * s + rank, 0.0, 1.0)
        N.call("ns_fill_normal", dev.handle, w.ptr, N.NS_F32, C.c_int64(NN * K), 2 + 16 * s, 0.0, 0.02)
        xq, xs, wq, ws = dev.empty(M * K, N.NS_I8), dev.empty(M), dev.empty(NN * K, N.NS_I8), dev.empty(NN)
        N.call("ns_quantize_rows_i8", dev.handle, x.ptr, N.NS_F32, C.c_int64(M), K, xq.ptr, xs.ptr)
        N.call("ns_quantize_rows_i8", dev.handle, w.ptr, N.NS_F32, C.c_int64(NN), K, wq.ptr, ws.ptr)
        bias = dev.empty(NN)
        N.call("ns_fill_normal", dev.handle, bias.ptr, N.NS_F32, C.c_int64(NN), 3 + 16 * s, 0.0, 0.01)
        y = dev.empty(M * NN)
        dev.synchronize()
        w.release()
        sets.append({"x": x, "xq": xq, "xs": xs, "wq": wq, "ws": ws, "bias": bias, "y": y})

    def step(i):
        t = sets[i % SETS]
        N.call("ns_qmatmul_i8", dev.handle, t["xq"].ptr, t["xs"].ptr, t["wq"].ptr, t["ws"].ptr, t["bias"].ptr, 0, 0, M, NN, K,
               N.EPI_BIAS, N.NS_F32, t["y"].ptr, 0)

    def barrier():
        dev.synchronize()
        if dist is not None:
            dist.barrier()
        dev.synchronize()

    def load_for(seconds):
        # untimed steps of the same workload, so that clock samples (every 200 ms) bracket the timed region
        t_end, i = time.time() + seconds, 0
        while time.time() < t_end:
            step(i); i += 1
            if i % 16 == 0:
                dev.synchronize()
        dev.synchronize()

    for i in range(args.warmup):
        step(i)
    e0, e1 = dev.event(), dev.event()
    sampler = ClockSampler(local_rank)
    dev.synchronize()
    if rank == 0:
        sampler.start()
    load_for(0.45)
    barrier()
    dev.record(e0)
    for i in range(args.steps):
        step(i)
    dev.record(e1)
    ms_total = dev.elapsed_ms(e0, e1)
    barrier()
    load_for(0.45)
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        import torch
        t = torch.tensor([ms_total], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * OPS / (ms_step * 1e-3) / 1e12

    # ---- end to end: pinned host float activations in, float result out, through the C ABI
    e2e_steps = max(3, min(args.steps, 8))
    hx, hy = C.c_void_p(), C.c_void_p()
    N.call("ns_host_alloc", C.c_uint64(M * K * 4), C.byref(hx))
    N.call("ns_host_alloc", C.c_uint64(M * NN * 4), C.byref(hy))
    t = sets[0]
    N.call("ns_d2h", dev.handle, hx, C.c_uint64(t["x"].ptr), C.c_uint64(M * K * 4))
    # the layer object a caller holds: made once from float [K, N] weights and a bias, as Linear keeps them
    w_f = dev.empty(NN * K)
    N.call("ns_fill_normal", dev.handle, w_f.ptr, N.NS_F32, C.c_int64(NN * K), 2, 0.0, 0.02)
    w_kn = np.ascontiguousarray(w_f.download((NN, K)).T)
    b_host = t["bias"].download()
    w_f.release()
    lin = C.c_void_p()
    N.call("ns_linear_create", dev.handle, K, NN, N.NS_I8, w_kn.ctypes.data_as(C.POINTER(C.c_float)),
           b_host.ctypes.data_as(C.POINTER(C.c_float)), N.SPLIT_NONE, 1, 0, 1, C.byref(lin))
    del w_kn

    def e2e_step(i):
        # one call: row chunks are uploaded, quantised, multiplied and downloaded on three overlapping streams
        N.call("ns_linear_forward_host", dev.handle, lin, hx, M, N.EPI_BIAS, hy, 0)

    e2e_step(0)
    barrier()
    dev.record(e0)
    for i in range(e2e_steps):
        e2e_step(i)
    dev.record(e1)
    e2e_ms = dev.elapsed_ms(e0, e1) / e2e_steps
    barrier()
    if dist is not None:
        import torch
        t2 = torch.tensor([e2e_ms], device=f"cuda:{local_rank}")
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e_ms = float(t2.item())
    e2e = {"value": world * OPS / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * NN * 4,
           "ms_per_step": e2e_ms, "steps": e2e_steps, "call": "ns_linear_forward_host (pinned float32 host buffers, three-stream row pipeline)",
           "link_gbs_each_way": M * K * 4 / (e2e_ms * 1e-3) / 1e9}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    achieved = OPS / (ms_step * 1e-3) / 1e12
    # The timed steps run inside about a second of back-to-back products (the clocks window), under the power cap:
    # the sustained figure is the denominator; the burst one and the nominal one are given beside it.
    int8_peak = 2.0 * peaks["bf16_sustained"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH, "kernel": "ns_gemm_pair_kernel<int8> (256 x 256 tiles, tcgen05 cta_group::2)",
                "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}; a kernel timed inside a long "
                               "loaded region, SM clock in `clocks`); that file has no int8 figure; nominal dense int8 is 4500",
                "frac_of_burst": achieved / (2.0 * peaks["bf16"]), "frac_of_nominal_4500": achieved / 4500.0,
                "algorithmic_bytes": ALGO_BYTES, "hbm_gbs_at_this_rate": ALGO_BYTES / (ms_step * 1e-3) / 1e9}
    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8",
           "data": "synthetic", "config": CONFIG, "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps, "roofline": roofline}
    if world == 1:
        tops, cores, secs = cpu_reference_tops(4096, 2)
        out["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port",
                               "sample": f"4096 of {M} rows, float32 product on de-quantised operands (how the float32-only reference "
                                         f"computes this Linear), best of 2, {secs:.2f} s each"}
    print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture summarised
# in profiles/.
TRAFFIC_BYTES_PER_LAUNCH = 149024512  # 63.85 MB read + 85.18 MB write, profiles/qmatmul_i8_m8192_k4096_n4096.md


def run_case(spec: str):
    """Small fixed cases for profiler captures (`ncu ... python bench.py --case NAME:ARGS`): three launches of one
    kernel on device-generated inputs, nothing timed.
      qmatmul_i8:M            int8 product, K = N = 4096, bias epilogue, f32 out
      qmatmul_i8_rows:M       int8 product of M <= 8 rows with 32768 x 8192 weights (268 MB, beyond L2): the row-streaming kernel
      attention_decode:L      batch 64, 32 heads, head_dim 128, cache length L
      attention_prefill:S     batch 8, 32 heads, head_dim 128, sequence S, causal
      gpt_decode:LAYERS       the int8 decoder of benchmark configuration 5 (d 2048, 16 heads, ff 8192, vocabulary 32000, batch 64)
                              cut to LAYERS layers: prompt of 512, then three decoding steps (seeded numpy weights);
                              prints the device time of a replayed step.  Under `python -m torch.distributed.run
                              --nproc-per-node N` the decoder is tensor-parallel over N GPUs (one rank per GPU, the
                              slowest rank's time is printed by rank 0)
    """
    import numpy as np
    from nn_b200 import native as N
    from nn_b200.device import Device
    name, _, arg = spec.partition(":")
    dev = Device(int(os.environ.get("LOCAL_RANK", "0")) if name == "gpt_decode" else 0)
    if name == "qmatmul_i8":
        m = int(arg or M)
        a, w = dev.empty(m * K, N.NS_I8), dev.empty(NN * K, N.NS_I8)
        N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_I8, C.c_int64(m * K), 1, 0.0, 40.0)
        N.call("ns_fill_normal", dev.handle, w.ptr, N.NS_I8, C.c_int64(NN * K), 9, 0.0, 40.0)
        a_s, w_s, b = dev.empty(m), dev.empty(NN), dev.empty(NN)
        for t, n_ in ((a_s, m), (w_s, NN), (b, NN)):
            N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_F32, C.c_int64(n_), 5, 1.0, 0.1)
        y = dev.empty(m * NN)
        for _ in range(3):
            N.call("ns_qmatmul_i8", dev.handle, a.ptr, a_s.ptr, w.ptr, w_s.ptr, b.ptr, 0, 0, m, NN, K, N.EPI_BIAS, N.NS_F32, y.ptr, 0)
    elif name == "qmatmul_i8_rows":
        m, n_, k_ = int(arg or 1), 32768, 8192
        a, w = dev.empty(m * k_, N.NS_I8), dev.empty(n_ * k_, N.NS_I8)
        N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_I8, C.c_int64(m * k_), 1, 0.0, 40.0)
        N.call("ns_fill_normal", dev.handle, w.ptr, N.NS_I8, C.c_int64(n_ * k_), 9, 0.0, 40.0)
        a_s, w_s, b = dev.empty(m), dev.empty(n_), dev.empty(n_)
        for t, cnt in ((a_s, m), (w_s, n_), (b, n_)):
            N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_F32, C.c_int64(cnt), 5, 1.0, 0.1)
        y = dev.empty(m * n_)
        for _ in range(3):
            N.call("ns_qmatmul_i8", dev.handle, a.ptr, a_s.ptr, w.ptr, w_s.ptr, b.ptr, 0, 0, m, n_, k_, N.EPI_BIAS, N.NS_F32, y.ptr, 0)
    elif name == "attention_decode":
        B, heads, dh, L, ps = 64, 32, 128, int(arg or 1024), 64
        max_pages = (L + ps) // ps
        h = C.c_void_p()
        N.call("ns_kv_cache_create", dev.handle, B * max_pages, ps, heads, dh, C.byref(h))
        kp, vp, nb = C.c_uint64(), C.c_uint64(), C.c_uint64()
        N.call("ns_kv_cache_pools", h, C.byref(kp), C.byref(vp), C.byref(nb))
        N.call("ns_fill_normal", dev.handle, kp.value, N.NS_BF16, C.c_int64(nb.value // 2), 2, 0.0, 1.0)
        N.call("ns_fill_normal", dev.handle, vp.value, N.NS_BF16, C.c_int64(nb.value // 2), 3, 0.0, 1.0)
        table = dev.from_numpy(np.arange(B * max_pages, dtype=np.int32))
        pos = dev.from_numpy(np.array([L - 1], np.int32))
        q, o = dev.empty(B * heads * dh, N.NS_BF16), dev.empty(B * heads * dh, N.NS_BF16)
        N.call("ns_fill_normal", dev.handle, q.ptr, N.NS_BF16, C.c_int64(B * heads * dh), 1, 0.0, 1.0)
        for _ in range(3):
            N.call("ns_attention_decode", dev.handle, h, q.ptr, C.c_int64(heads * dh), o.ptr, C.c_int64(heads * dh), table.ptr, max_pages,
                   pos.ptr, B, 1, C.c_float(0.0884))
    elif name == "attention_prefill":
        B, H, S = 8, 32, int(arg or 2048)
        n = B * H * S * 128
        q, k, v, o = (dev.empty(n, N.NS_BF16) for _ in range(4))
        for t, seed in ((q, 1), (k, 2), (v, 3)):
            N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_BF16, C.c_int64(n), seed, 0.0, 1.0)
        st = (C.c_int64 * 3)(H * S * 128, S * 128, 128)
        for _ in range(3):
            N.call("ns_attention_prefill", dev.handle, q.ptr, k.ptr, v.ptr, o.ptr, B, H, S, 128, st, st, st, st, C.c_float(0.0884), 1)
    elif name == "gpt_decode":
        from nn_b200.gpt import GptConfig, GptW8A8
        layers, B, prompt_len = int(arg or 2), 64, 512
        cfg = GptConfig(vocab=32000, dim=2048, heads=16, layers=layers, ff_dim=8192, context=768)
        rng = np.random.default_rng(4)
        D, FF, V = cfg.dim, cfg.ff_dim, cfg.vocab
        nrm = lambda *shape, s=0.02: (rng.standard_normal(shape, dtype=np.float32) * s)
        w = {"tok": nrm(V, D), "pos": nrm(cfg.context, D), "lnf_g": 1.0 + nrm(D, s=0.05), "lnf_b": nrm(D), "head_w": nrm(D, V), "head_b": nrm(V, s=0.01),
             "l0.ln1_g": 1.0 + nrm(D, s=0.05), "l0.ln1_b": nrm(D), "l0.ln2_g": 1.0 + nrm(D, s=0.05), "l0.ln2_b": nrm(D),
             "l0.qkv_w": nrm(D, 3 * D), "l0.qkv_b": nrm(3 * D, s=0.01), "l0.out_w": nrm(D, D), "l0.out_b": nrm(D, s=0.01),
             "l0.ff1_w": nrm(D, FF), "l0.ff1_b": nrm(FF, s=0.01), "l0.ff2_w": nrm(FF, D), "l0.ff2_b": nrm(D, s=0.01)}
        from nn_b200 import dist
        comm, rank, world = dist.init_comm(dev)
        model = GptW8A8(dev, cfg, w, B, max_prefill=prompt_len, share_layer_weights=True, tp_rank=rank, tp_size=world,
                        comm=comm)   # every layer its own device copy
        model.prefill(rng.integers(0, V, (B, prompt_len)).astype(np.int32))
        for _ in range(3):
            model.step(False)
        dev.synchronize()
        e0, e1 = dev.event(), dev.event()
        model.step(True)
        model.step(True)
        dev.record(e0)
        for _ in range(20):
            model.step(True)
        dev.record(e1)
        ms = dist.all_reduce_max(dev.elapsed_ms(e0, e1) / 20)
        dev.synchronize()
        launches = model.launches_per_step
        model.close()
        if rank == 0:
            print(json.dumps({"case": spec, "ok": True, "ms_per_replayed_step": ms, "tokens_per_s": B / ms * 1e3, "layers": layers,
                              "tensor_parallel": world, "launches_per_step": launches}))
        return
    else:
        raise SystemExit(f"unknown case {spec}")
    dev.synchronize()
    print(json.dumps({"case": spec, "ok": True}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="profiler case, see run_case")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.warmup < 3:
        args.warmup = 3
    if args.case:
        run_case(args.case)
    elif args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
