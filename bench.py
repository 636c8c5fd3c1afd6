"""Benchmark of the hot path: int8 QuantizedMatMul (int8 x int8 -> int32, per-channel dequant + bias epilogue), and the
int8 GPT decoder's greedy generation (tokens/s), tensor-parallel over the GPUs of the run.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-gpt]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Headline workload (benchmark configuration "int8 QuantizedMatMul sweep", the largest M): A [8192, 4096] float ~N(0,1)
quantised per row, W [4096, 4096] ~N(0,0.02) quantised per output channel, bias ~N(0,0.01), float output.  One step =
one pass of the product over one batch of 8192 rows.  With N > 1 GPUs every rank runs its own batch of rows against
its own copy of the weights (batch sharding, no data-path collective): weak scaling.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput, `e2e` is the same product through the C ABI
from pinned host buffers (float activations in, float result out, copies inside the timed region), `roofline`
compares the tcgen05 kernel with the tensor-core peak, `cpu_baseline` times the oracle's restatement of the
reference's CPU product on this host's cores.  `gpt_decode` is the second half of the metric: the 24-layer int8
decoder (d 2048, 16 heads, FF 8192, vocabulary 32000), batch 64, prompt 512, 256 greedy tokens, tensor-parallel over
the N ranks, after a 40-token warm-up generation (the reference's harness does the same:
samples/NeuralSharp.Samples.Transformer/Program.cs:122-142; tokens/s over all sequences, samples/Shared/Gpt/
CharGpt.cs:321-333); on rank 0 the same model also runs on one GPU and the tokens are compared.
`--impl reference` times the CPU restatement alone (the reference is C#/.NET and cannot run here).
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
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, NN = 8192, 4096, 4096
OPS = 2.0 * M * K * NN
ALGO_BYTES = NN * K + M * K + 4 * M * NN + 4 * (M + 2 * NN)
METRIC, UNIT = "int8_quantized_matmul_tops", "TOPS"
MIN_TIMED_SECONDS = 0.35      # the timed region is stretched to at least this (a 200 ms clock sampler must see it)
CONFIG = {"workload": "int8 QuantizedMatMul M=8192 K=4096 N=4096 (per-row A scales, per-channel W scales, bias, f32 out)",
          "l2": "4 operand/result sets rotated per step (704 MB footprint > 126 MB L2)", "seed": 1,
          "clocks_window": "nvidia-smi sampled every 200 ms over the loaded region: 0.45 s of untimed steps, the timed steps "
                           "(at least 0.35 s), 0.45 s of untimed steps"}

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture summarised
# in profiles/.
TRAFFIC_BYTES_PER_LAUNCH = 146382848  # 61.31 MB read + 85.08 MB write, profiles/qmatmul_i8_m8192_k4096_n4096.md


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

    def __init__(self, gpu_index: int, tag: str = ""):
        self.gpu_index, self.proc, self.path = gpu_index, None, f"/tmp/ns_b200_clocks_{os.getpid()}{tag}.csv"

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


# ---------------------------------------------------------------------------------------------------------------
# the decoder of benchmark configuration 5
# ---------------------------------------------------------------------------------------------------------------
GPT = {"vocab": 32000, "dim": 2048, "heads": 16, "layers": 24, "ff_dim": 8192, "batch": 64, "prompt": 512, "new_tokens": 256,
       "warmup_tokens": 40, "seed": 4}


class SyntheticGptWeights(dict):
    """The weight mapping GptW8A8 takes, produced tensor by tensor on first use and not kept: matrices ~N(0, 0.02)
    (the benchmark configuration's rule), LayerNorm gains 1 + N(0, 0.05), biases N(0, 0.01).  The stream of a tensor depends on
    (seed, its key) only, so every rank of a tensor-parallel run cuts its shards from identical matrices."""

    def __init__(self, cfg, seed: int):
        super().__init__()
        self.cfg, self.seed = cfg, seed

    def _shape(self, name: str):
        c = self.cfg
        D, FF, V = c.dim, c.ff_dim, c.vocab
        table = {"tok": (V, D), "pos": (c.context, D), "lnf_g": (D,), "lnf_b": (D,), "head_w": (D, V), "head_b": (V,),
                 "ln1_g": (D,), "ln1_b": (D,), "ln2_g": (D,), "ln2_b": (D,), "qkv_w": (D, 3 * D), "qkv_b": (3 * D,), "out_w": (D, D),
                 "out_b": (D,), "ff1_w": (D, FF), "ff1_b": (FF,), "ff2_w": (FF, D), "ff2_b": (D,)}
        return table[name]

    def __getitem__(self, key: str):
        name = key.split(".")[-1]
        shape = self._shape(name)
        rng = np.random.default_rng([self.seed, zlib.crc32(key.encode())])
        x = rng.standard_normal(shape, dtype=np.float32)
        if name.endswith("_g"):
            x *= 0.05
            x += 1.0
        elif name.endswith("_b") and len(shape) == 1 and name not in ("ln1_b", "ln2_b", "lnf_b"):
            x *= 0.01
        else:
            x *= 0.02
        return x


def gpt_prompt(cfg, batch: int, length: int, seed: int) -> np.ndarray:
    return np.random.default_rng([seed, 7]).integers(0, cfg.vocab, (batch, length)).astype(np.int32)


def decode_step_bytes(cfg, batch: int, context: float, gpus: int) -> float:
    """Algorithmic HBM bytes of one decoding step per GPU: int8 weights of every Linear once + the cached keys and values
    of `context` positions (bf16), both sharded over the GPUs."""
    D, FF, V, L = cfg.dim, cfg.ff_dim, cfg.vocab, cfg.layers
    weights = L * (D * 3 * D + D * D + 2 * D * FF) + D * V
    kv = L * 2 * batch * context * D * 2
    return (weights + kv) / gpus


def run_gpt_decode(dev, rank: int, world: int, peaks: dict, layers: int, new_tokens: int, compare_tp1: bool, fused: int | None = None,
                   attn_quant: bool | None = None, batch: int | None = None, unfused_rows: int | None = None):
    """Builds the decoder tensor-parallel over the ranks of the run, warms up, times one generation; returns the
    `gpt_decode` record on rank 0 (None elsewhere)."""
    from nn_b200 import dist as nsdist
    from nn_b200.gpt import GptConfig, GptW8A8

    g = GPT
    B, P = batch or g["batch"], g["prompt"]
    cfg = GptConfig(vocab=g["vocab"], dim=g["dim"], heads=g["heads"], layers=layers, ff_dim=g["ff_dim"], context=P + g["new_tokens"])
    weights = SyntheticGptWeights(cfg, g["seed"])
    prompt = gpt_prompt(cfg, B, P, g["seed"])
    comm = None
    if world > 1:
        comm, _, _ = nsdist.init_comm(dev)
    t0 = time.perf_counter()
    model = GptW8A8(dev, cfg, weights, B, max_prefill=P, tp_rank=rank, tp_size=world, comm=comm)
    if fused is not None:
        model.fused = fused
    if attn_quant is not None:
        model.attn_quant = attn_quant
    if unfused_rows is not None:
        model.unfused_rows = unfused_rows
    if world > 1:
        # the prompt is read by batch sharding (a full copy of the weights per GPU), decoding is tensor-parallel
        model.enable_batch_sharded_prefill(weights)
    build_s = time.perf_counter() - t0

    warm_tokens, _ = model.generate(prompt, min(g["warmup_tokens"], new_tokens))   # warm-up generation: sizes scratch, records the step graph
    dev.synchronize()
    nsdist.barrier()
    sampler = ClockSampler(dev.ordinal, "_gpt")
    if rank == 0:
        sampler.start()
    marks = {}
    wall0 = time.perf_counter()
    tokens, resets = model.generate(prompt, new_tokens, marks=marks)
    dev.synchronize()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else None
    prefill_ms = nsdist.all_reduce_max(dev.elapsed_ms(marks["start"], marks["prefill_end"]))
    steps = marks["steps"]
    decode_ms = nsdist.all_reduce_max(dev.elapsed_ms(marks["prefill_end"], steps[-1][1]))
    n_steps = new_tokens - 1
    seg = []
    prev_count, prev_event = 1, marks["prefill_end"]
    for count, ev in steps:
        seg.append((prev_count, count, nsdist.all_reduce_max(dev.elapsed_ms(prev_event, ev)) / max(1, count - prev_count)))
        prev_count, prev_event = count, ev
    ms_step = decode_ms / n_steps
    launches = model.launches_per_step

    # the step with the cross-GPU exchange in its single-rank form (results are not the model's): what the exchange costs
    exchange = None
    if world > 1 and model.peer is not None:
        def replay_ms(n=48):
            model.prefill(prompt)
            for _ in range(3):
                model.step(True)
            e0, e1 = dev.event(), dev.event()
            dev.synchronize()
            nsdist.barrier()
            dev.record(e0)
            for _ in range(n):
                model.step(True)
            dev.record(e1)
            return nsdist.all_reduce_max(dev.elapsed_ms(e0, e1) / n)
        full = replay_ms()
        model.set_local_exchange(True)
        local = replay_ms()
        model.set_local_exchange(False)
        exchange = {"ms_per_step_full": full, "ms_per_step_single_rank_exchange": local, "exchange_ms_per_step": full - local,
                    "context": f"{P}+3..{P}+51"}
    # the alternative partition: pure batch sharding -- every GPU decodes batch / N sequences with the full weights, no
    # exchange at all (the one-GPU model each rank already holds for the prompt read)
    alt, alt_tokens = None, None
    if world > 1 and model.replica is not None:
        rep, bl = model.replica, B // world
        sub = prompt[rank * bl:(rank + 1) * bl]
        rep.generate(sub, min(g["warmup_tokens"], new_tokens))
        dev.synchronize()
        nsdist.barrier()
        m2 = {}
        toks, _ = rep.generate(sub, new_tokens, marks=m2)
        dev.synchronize()
        p_ms = nsdist.all_reduce_max(dev.elapsed_ms(m2["start"], m2["prefill_end"]))
        d_ms = nsdist.all_reduce_max(dev.elapsed_ms(m2["prefill_end"], m2["steps"][-1][1]))
        gathered = nsdist.all_gather_bytes(np.ascontiguousarray(toks, np.int32).tobytes())
        alt_tokens = np.concatenate([np.frombuffer(x, np.int32).reshape(bl, new_tokens) for x in gathered], axis=0)
        alt = {"parallelism": f"batch sharding: {world} x {bl} sequences, full weights per GPU, no exchange",
               "tokens_per_s": B * n_steps / (d_ms * 1e-3), "prefill_ms": p_ms, "ms_per_step": d_ms / n_steps, "launches_per_step": rep.launches_per_step,
               "hbm_frac": (decode_step_bytes(cfg, B, P + new_tokens / 2.0, 1) - (1.0 - 1.0 / world) * cfg.layers * 2 * B * (P + new_tokens / 2.0) * cfg.dim * 2)
                           / (d_ms / n_steps * 1e-3) / 1e9 / peaks["hbm"]}
    prefill_mode = "batch sharding + key/value delivery over peer memory" if model.replica is not None else "same partition as decoding"
    model.close()
    nsdist.barrier()

    # the same model on one GPU (rank 0), tokens compared step by step
    compare = None
    if rank == 0:
        if world == 1:
            compare = {"tokens_equal_tp1_prefix": new_tokens, "note": "this run is the one-GPU model"}
        elif compare_tp1:
            one = GptW8A8(dev, cfg, weights, B, max_prefill=P)
            ref_tokens, _ = one.generate(prompt, new_tokens)
            same = np.all(ref_tokens == tokens, axis=0)
            prefix = int(np.argmin(same)) if not same.all() else new_tokens
            compare = {"tokens_equal_tp1_prefix": prefix, "of_steps": new_tokens,
                       "sequences_equal_throughout": int(np.all(ref_tokens == tokens, axis=1).sum()), "of_sequences": B}
            if alt_tokens is not None:
                same_alt = np.all(ref_tokens == alt_tokens, axis=0)
                alt["tokens_equal_tp1_prefix"] = int(np.argmin(same_alt)) if not same_alt.all() else new_tokens
                alt["sequences_equal_throughout"] = int(np.all(ref_tokens == alt_tokens, axis=1).sum())
            if prefix < new_tokens:
                b = int(np.argmax(ref_tokens[:, prefix] != tokens[:, prefix]))
                one.generate(prompt, prefix + 1)                       # deterministic: ends on the step that produced token `prefix`
                dev.synchronize()
                row = one.read_logits()[b]
                top = np.sort(row)[-2:]
                tol = 2 * 5e-2 * max(1.0, abs(float(top[1])))
                compare["first_departure"] = {"step": prefix, "sequence": b, "tp1_token": int(ref_tokens[b, prefix]), "tpN_token": int(tokens[b, prefix]),
                                              "tp1_top2_gap": float(top[1] - top[0]), "near_tie_tolerance": tol,
                                              "is_near_tie": bool(top[1] - top[0] <= tol),
                                              "tpN_token_logit_below_top": float(top[1] - row[int(tokens[b, prefix])])}
            one.close()
    nsdist.barrier()
    if rank != 0:
        return None
    mean_ctx = P + (new_tokens / 2.0)
    step_bytes = decode_step_bytes(cfg, B, mean_ctx, world)
    rec = {"config": {"model": f"int8 GPT decoder, {layers} layers, d {cfg.dim}, {cfg.heads} heads, ff {cfg.ff_dim}, vocabulary {cfg.vocab}",
                      "batch": B, "prompt": P, "new_tokens": new_tokens, "warmup_tokens": min(g["warmup_tokens"], new_tokens),
                      "parallelism": f"tp{world}" if world > 1 else "1 gpu",
                      "weights": "synthetic, seeded per tensor, every layer its own values", "seed": g["seed"]},
           "tokens_per_s": B * n_steps / (decode_ms * 1e-3), "tokens_per_s_wall_incl_prefill": B * new_tokens / wall,
           "prefill_ms": prefill_ms, "prefill_mode": prefill_mode, "prefill_tokens_per_s": B * P / (prefill_ms * 1e-3), "decode_ms": decode_ms,
           "ms_per_step": ms_step,
           "ms_per_step_first_segment": seg[0][2], "ms_per_step_last_segment": seg[-1][2],
           "segments": [{"tokens": [a, b], "ms_per_step": ms} for a, b, ms in seg],
           "launches_per_step": launches, "context_resets": resets,
           "hbm_bytes_per_step_per_gpu": step_bytes, "hbm_frac": step_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm"],
           "hbm_peak_gbs": peaks["hbm"], "clocks": clocks, "model_build_s": build_s, "exchange": exchange, "batch_sharded_decode": alt,
           "tokens_equal_on_repeat": bool(np.array_equal(warm_tokens, tokens[:, :warm_tokens.shape[1]]))}
    if compare is not None:
        rec.update(compare)
    return rec


def bind_near_gpu(gpu_index: int):
    """Restricts this process to the host cores NVML lists as local to the GPU (when that is a proper subset of what it may
    use), so that pinned buffers allocated next land on the GPU's NUMA node.  Returns (old affinity, note)."""
    old = os.sched_getaffinity(0)
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        pynvml.nvmlShutdown()
    except Exception as e:   # NVML missing or not permitted: stay as we are
        return old, f"NVML affinity unavailable ({type(e).__name__})"
    both = near & old
    if both and both != old:
        os.sched_setaffinity(0, both)
        return old, f"bound to {len(both)} GPU-local cores of {len(old)}"
    return old, f"GPU-local cores = all {len(old)} usable cores (one NUMA node visible)"


def run_ours(args, rank, world, local_rank):
    from nn_b200 import native as N
    from nn_b200.device import Device

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        # gloo for host-side rendezvous (NCCL ids, IPC handles), NCCL for barriers and the max over ranks
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local_rank))
    dev = Device(local_rank)
    peaks = measured_peaks()

    def barrier():
        dev.synchronize()
        if dist is not None:
            import torch
            t = torch.zeros(1, device=f"cuda:{local_rank}")
            dist.all_reduce(t)
            torch.cuda.synchronize()
        dev.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    barrier()      # throw-away: the first collective sets up the communicator; later barriers take microseconds

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
        if s > 0:
            x.release()
        sets.append({"x": x, "xq": xq, "xs": xs, "wq": wq, "ws": ws, "bias": bias, "y": y})

    def step(i):
        t = sets[i % SETS]
        N.call("ns_qmatmul_i8", dev.handle, t["xq"].ptr, t["xs"].ptr, t["wq"].ptr, t["ws"].ptr, t["bias"].ptr, 0, 0, M, NN, K,
               N.EPI_BIAS, N.NS_F32, t["y"].ptr, 0)

    def load_for(seconds):
        # untimed steps of the same workload, so that clock samples (every 200 ms) bracket the timed region
        t_end, i = time.time() + seconds, 0
        while time.time() < t_end:
            step(i); i += 1
            if i % 16 == 0:
                dev.synchronize()
        dev.synchronize()

    e0, e1 = dev.event(), dev.event()
    for i in range(args.warmup):
        step(i)
    # a first estimate of the step time sizes the timed region: the K steps asked for, and as many more as it takes
    # for the region to last MIN_TIMED_SECONDS
    dev.synchronize()
    dev.record(e0)
    for i in range(20):
        step(i)
    dev.record(e1)
    est_ms = max(dev.elapsed_ms(e0, e1) / 20, 1e-3)
    executed = args.steps if args.short else max(args.steps, int(MIN_TIMED_SECONDS * 1e3 / est_ms) + 1)
    executed = int(max_over_ranks(float(executed)))
    sampler = ClockSampler(local_rank)
    dev.synchronize()
    if rank == 0:
        sampler.start()
    load_for(0.0 if args.short else 0.45)
    barrier()
    dev.record(e0)
    for i in range(executed):
        step(i)
    dev.record(e1)
    ms_total = dev.elapsed_ms(e0, e1)
    barrier()
    load_for(0.0 if args.short else 0.45)
    clocks = sampler.stop() if rank == 0 else None
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / executed
    value = world * OPS / (ms_step * 1e-3) / 1e12

    # ---- the main loop alone (loads + MMAs of the same pair kernel, nothing dequantised or written), K = 16384: the int8
    # rate this library's pipeline reaches, as a measured yardstick beside 2 x the cuBLAS bf16 figure
    KP = 16384
    pa, pw = dev.empty(M * KP, N.NS_I8), dev.empty(NN * KP, N.NS_I8)
    N.call("ns_fill_normal", dev.handle, pa.ptr, N.NS_I8, C.c_int64(M * KP), 21, 0.0, 40.0)
    N.call("ns_fill_normal", dev.handle, pw.ptr, N.NS_I8, C.c_int64(NN * KP), 22, 0.0, 40.0)
    for _ in range(3):
        N.call("ns_bench_i8_mainloop", dev.handle, pa.ptr, pw.ptr, M, NN, KP)
    n_proxy = 3 if args.short else 200
    barrier()
    dev.record(e0)
    for _ in range(n_proxy):
        N.call("ns_bench_i8_mainloop", dev.handle, pa.ptr, pw.ptr, M, NN, KP)
    dev.record(e1)
    proxy_tops = 2.0 * M * KP * NN / (dev.elapsed_ms(e0, e1) / n_proxy * 1e-3) / 1e12
    barrier()
    pa.release(); pw.release()

    # ---- end to end: pinned host float activations in, float result out, through the C ABI
    e2e_steps = max(3, min(args.steps, 8))
    old_affinity, affinity_note = bind_near_gpu(local_rank)
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
    e2e_ms = max_over_ranks(e2e_ms)
    # the host link alone, every rank at once: uploads of the same pinned buffer, nothing else
    barrier()
    dev.record(e0)
    for i in range(4):
        N.call("ns_h2d_async", dev.handle, C.c_uint64(t["x"].ptr), hx, C.c_uint64(M * K * 4))
    dev.record(e1)
    h2d_ms = max_over_ranks(dev.elapsed_ms(e0, e1) / 4)
    barrier()
    os.sched_setaffinity(0, old_affinity)
    e2e = {"value": world * OPS / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * NN * 4,
           "ms_per_step": e2e_ms, "steps": e2e_steps, "call": "ns_linear_forward_host (pinned float32 host buffers, three-stream row pipeline)",
           "link_gbs_each_way": M * K * 4 / (e2e_ms * 1e-3) / 1e9,
           "h2d_alone_gbs_per_gpu": M * K * 4 / (h2d_ms * 1e-3) / 1e9, "h2d_alone_gbs_all_gpus": world * M * K * 4 / (h2d_ms * 1e-3) / 1e9,
           "host_affinity": affinity_note}
    N.call("ns_linear_destroy", lin)
    N.call("ns_host_free", hx)
    N.call("ns_host_free", hy)
    for tset in sets:
        for st in tset.values():
            st.release()
    sets.clear()

    # ---- the decoder: tokens/s of a greedy generation, tensor-parallel over the ranks
    gpt = None
    if not args.no_gpt:
        gpt = run_gpt_decode(dev, rank, world, peaks, args.gpt_layers, args.gpt_tokens, compare_tp1=not args.no_tp1)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    achieved = OPS / (ms_step * 1e-3) / 1e12
    # Denominator: MEASURED_PEAKS.json has no int8 figure, so 2 x the cuBLAS bf16 rate.  Its burst figure was taken at the
    # clock a tensor-core load holds for a short while (~1.45 GHz), the sustained one at ~1.35 GHz under the power cap:
    # the line's own median SM clock says which regime the timed steps ran in.
    sm = clocks.get("sm_mhz") if clocks else None
    use_sustained = sm is not None and sm <= 1380.0
    int8_peak = 2.0 * (peaks["bf16_sustained"] if use_sustained else peaks["bf16"])
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH, "kernel": "ns_gemm_pair_kernel<int8> (256 x 256 tiles, tcgen05 cta_group::2)",
                "peak_source": ("2 x bf16_tflops_sustained" if use_sustained else "2 x bf16_tflops (burst)") +
                               f" of MEASURED_PEAKS.json ({peaks['source']}): median SM clock of the loaded region {sm} MHz "
                               + ("<= 1380" if use_sustained else "> 1380") + "; that file has no int8 figure; nominal dense int8 is 4500",
                "frac_of_burst": achieved / (2.0 * peaks["bf16"]), "frac_of_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
                "frac_of_nominal_4500": achieved / 4500.0,
                "i8_mainloop_proxy_tops": proxy_tops, "frac_of_i8_proxy": achieved / proxy_tops,
                "i8_mainloop_proxy": f"ns_bench_i8_mainloop M={M} N={NN} K={KP}, {n_proxy} launches: loads + MMAs only, nothing written",
                "algorithmic_bytes": ALGO_BYTES, "hbm_gbs_at_this_rate": ALGO_BYTES / (ms_step * 1e-3) / 1e9}
    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "steps_executed": executed,
           "timed_region_s": ms_total * 1e-3, "warmup": args.warmup,
           "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8",
           "data": "synthetic", "config": CONFIG, "clocks": clocks, "e2e": e2e, "gpu_launches": executed, "roofline": roofline}
    if gpt is not None:
        out["gpt_decode"] = gpt
    if world == 1:
        tops, cores, secs = cpu_reference_tops(4096, 2)
        out["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port",
                               "sample": f"4096 of {M} rows, float32 product on de-quantised operands (how the float32-only reference "
                                         f"computes this Linear), best of 2, {secs:.2f} s each"}
    print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def run_case(spec: str):
    """Small fixed cases for profiler captures (`ncu ... python bench.py --case NAME:ARGS`): three launches of one
    kernel on device-generated inputs, nothing timed unless stated.
      qmatmul_i8:M            int8 product, K = N = 4096, bias epilogue, f32 out
      qmatmul_i8_rows:M       int8 product of M <= 8 rows with 32768 x 8192 weights (268 MB, beyond L2): the row-streaming kernel
      i8_mainloop_peak[:K]    the pair kernel's main loop alone (ns_bench_i8_mainloop), M = 8192, N = 4096, K = 16384 unless given:
                              prints the TOPS of 200 timed launches -- the int8 tensor-core rate the load / MMA pipeline reaches
      second_phase_times      ns_linear_forward_norm_quant / _gelu_quant at 64 rows: per-CTA times of the kernel's phases (product done,
                              all CTAs arrived, rows done) from the library's timing hook, and the time per call
      decode_shapes           the weight-streaming products (int8 M in {1, 16, 128} at K = N = 4096; bf16 M = 8, K = 4096, N = 14336;
                              the five M = 64 products of the decoder step) timed as graphs of 20 launches over weight copies
                              beyond L2, beside the same graph of an empty kernel: prints time, GB/s and fraction of the HBM peak
      attention_decode:L      batch 64, 32 heads, head_dim 128, cache length L
      attention_prefill:S     batch 8, 32 heads, head_dim 128, sequence S, causal
      prefill_parts           one decoder layer of the prompt read of benchmark configuration 5 (32768 rows), operator by operator: time,
                              bytes and GB/s (row kernels) or TOPS (products, attention) of each
      gpt_decode:LAYERS[:T[:F[:Q[:B[:U]]]]] the int8 decoder of benchmark configuration 5 (d 2048, 16 heads, ff 8192, vocabulary 32000, batch 64,
                              prompt 512) cut to LAYERS layers, T new tokens (default 64): prints the gpt_decode record
                              of the default run.  Under `python -m torch.distributed.run --nproc-per-node N` the decoder
                              is tensor-parallel over N GPUs (one rank per GPU, the slowest rank's times are printed by rank 0).
                              F picks the few-row pass: 2 one launch per Linear, 1 product + fused row kernel, 0 one kernel per operator;
                              Q = 0 keeps the row quantisation after attention a kernel of its own; B = batch instead of 64; U = passes of up to U
                              rows take one kernel per operator
    """
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
    elif name == "i8_mainloop_peak":
        kp = int(arg or 16384)
        a, w = dev.empty(M * kp, N.NS_I8), dev.empty(NN * kp, N.NS_I8)
        N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_I8, C.c_int64(M * kp), 1, 0.0, 40.0)
        N.call("ns_fill_normal", dev.handle, w.ptr, N.NS_I8, C.c_int64(NN * kp), 9, 0.0, 40.0)
        for _ in range(3):
            N.call("ns_bench_i8_mainloop", dev.handle, a.ptr, w.ptr, M, NN, kp)
        e0, e1 = dev.event(), dev.event()
        dev.synchronize()
        dev.record(e0)
        for _ in range(200):
            N.call("ns_bench_i8_mainloop", dev.handle, a.ptr, w.ptr, M, NN, kp)
        dev.record(e1)
        us = dev.elapsed_ms(e0, e1) / 200 * 1e3
        print(json.dumps({"case": spec, "ok": True, "us_per_launch": us, "tops": 2.0 * M * kp * NN / (us * 1e-6) / 1e12, "M": M, "N": NN, "K": kp}))
        return
    elif name == "second_phase_times":
        # One launch per Linear (ns_linear_forward_norm_quant / _gelu_quant): where the time of the product kernel's second phase
        # goes.  Every CTA records four times (test hook ns_debug_tail_times): kernel start, product done (its stores
        # complete), every CTA arrived, rows done.  Weights stay the same from call to call (L2-resident).
        rng = np.random.default_rng(6)
        rows_m = 64
        times = dev.zeros(148 * 4 * 2, N.NS_I32)
        out = []
        for (k_, n_, kind) in [(2048, 2048, "norm"), (8192, 2048, "norm"), (2048, 8192, "gelu")]:
            w = rng.standard_normal((k_, n_), dtype=np.float32) * 0.05
            bvec = rng.standard_normal(n_, dtype=np.float32) * 0.1
            lin = C.c_void_p()
            N.call("ns_linear_create", dev.handle, k_, n_, N.NS_I8, w.ctypes.data_as(C.POINTER(C.c_float)), bvec.ctypes.data_as(C.POINTER(C.c_float)),
                   N.SPLIT_NONE, 1, 0, 1, C.byref(lin))
            x = dev.from_numpy(rng.standard_normal((rows_m, k_), dtype=np.float32))
            xq, xs = dev.empty(rows_m * k_, N.NS_I8), dev.empty(rows_m)
            N.call("ns_quantize_rows_i8", dev.handle, x.ptr, N.NS_F32, C.c_int64(rows_m), k_, xq.ptr, xs.ptr)
            res = dev.empty(rows_m * n_, N.NS_BF16)
            N.call("ns_fill_normal", dev.handle, res.ptr, N.NS_BF16, C.c_int64(rows_m * n_), 8, 0.0, 1.0)
            gam, bet = dev.from_numpy(np.ones(n_, np.float32)), dev.from_numpy(np.zeros(n_, np.float32))
            y, q, sc = dev.empty(rows_m * n_, N.NS_BF16), dev.empty(rows_m * max(n_, k_), N.NS_I8), dev.empty(rows_m)

            def call():
                if kind == "norm":
                    N.call("ns_linear_forward_norm_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), res.ptr, C.c_int64(rows_m), y.ptr,
                           gam.ptr, bet.ptr, C.c_float(1e-5), q.ptr, sc.ptr)
                else:
                    N.call("ns_linear_forward_gelu_quant", dev.handle, lin, C.c_uint64(xq.ptr), C.c_uint64(xs.ptr), C.c_int64(rows_m), q.ptr, sc.ptr)
            for _ in range(5):
                call()
            dev.synchronize()
            N.call("ns_debug_tail_times", dev.handle, C.c_uint64(times.ptr))
            call()
            dev.synchronize()
            N.call("ns_debug_tail_times", dev.handle, C.c_uint64(0))
            t = times.download().view(np.uint64).reshape(-1, 4).astype(np.int64)
            t = t[t[:, 0] > 0]
            rel = (t - t[:, 0].min()) / 1000.0
            waited = rel[rel[:, 3] > 0]
            e0, e1 = dev.event(), dev.event()
            dev.record(e0)
            for _ in range(50):
                call()
            dev.record(e1)
            out.append({"kind": kind, "M": rows_m, "K": k_, "N": n_, "ctas": int(len(t)), "row_ctas": int(len(waited)),
                        "product_done_us": [float(rel[:, 1].min()), float(rel[:, 1].max())],
                        "all_arrived_us": [float(rel[rel[:, 2] > 0][:, 2].min()), float(rel[:, 2].max())],
                        "rows_done_us": [float(waited[:, 3].min()), float(waited[:, 3].max())],
                        "us_per_call_back_to_back": dev.elapsed_ms(e0, e1) / 50 * 1e3})
            N.call("ns_memset32_async", dev.handle, C.c_uint64(times.ptr), 0, C.c_uint64(148 * 8))
            dev.synchronize()
            N.call("ns_linear_destroy", lin)
        print(json.dumps({"case": spec, "ok": True, "phases": out}))
        return
    elif name == "decode_shapes":
        # The weight-streaming products of the benchmark configurations, each as a graph of 20 launches over rotating weight copies
        # (more than the 126 MB of L2 in total, so every launch streams from HBM), and the same graph of an empty kernel
        # (ns_add_i32 of one thread): the launch floor a product of a few microseconds sits on.
        peaks = measured_peaks()
        reps = 20
        e0, e1 = dev.event(), dev.event()

        def timed_graph(launch):
            for i in range(reps):
                launch(i)
            dev.synchronize()
            dev.capture_begin()
            for i in range(reps):
                launch(i)
            g = dev.capture_end()
            for _ in range(3):
                dev.graph_launch(g)
            dev.synchronize()
            best = None
            for _ in range(5):
                dev.record(e0)
                dev.graph_launch(g)
                dev.record(e1)
                us = dev.elapsed_ms(e0, e1) / reps * 1e3
                best = us if best is None else min(best, us)
            dev.graph_destroy(g)
            return best

        counter = dev.zeros(1, N.NS_I32)
        floor_us = timed_graph(lambda i: N.call("ns_add_i32", dev.handle, counter.ptr, 0))
        rows = []
        shapes = [("i8", 1, 4096, 4096), ("i8", 16, 4096, 4096), ("i8", 128, 4096, 4096), ("bf16", 8, 14336, 4096),
                  ("i8", 64, 6144, 2048), ("i8", 64, 2048, 2048), ("i8", 64, 8192, 2048), ("i8", 64, 2048, 8192), ("i8", 64, 32000, 2048)]
        for kind, m, n_, k_ in shapes:
            el = 1 if kind == "i8" else 2
            copies = max(2, min(reps, -(-160_000_000 // (n_ * k_ * el))))
            ws = []
            for c in range(copies):
                w = dev.empty(n_ * k_, N.NS_I8 if kind == "i8" else N.NS_BF16)
                N.call("ns_fill_normal", dev.handle, w.ptr, N.NS_I8 if kind == "i8" else N.NS_BF16, C.c_int64(n_ * k_), 9 + c, 0.0, 40.0 if kind == "i8" else 1.0)
                ws.append(w)
            if kind == "i8":
                a = dev.empty(m * k_, N.NS_I8)
                N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_I8, C.c_int64(m * k_), 1, 0.0, 40.0)
                a_s, w_s, b = dev.empty(m), dev.empty(n_), dev.empty(n_)
                for t, cnt in ((a_s, m), (w_s, n_), (b, n_)):
                    N.call("ns_fill_normal", dev.handle, t.ptr, N.NS_F32, C.c_int64(cnt), 5, 1.0, 0.1)
                y = dev.empty(m * n_)
                us = timed_graph(lambda i: N.call("ns_qmatmul_i8", dev.handle, a.ptr, a_s.ptr, ws[i % copies].ptr, w_s.ptr, b.ptr, 0, 0, m, n_, k_,
                                                  N.EPI_BIAS, N.NS_F32, y.ptr, 0))
                nbytes = n_ * k_ + m * k_ + 4 * m * n_ + 4 * (m + 2 * n_)
            else:
                a = dev.empty(m * k_, N.NS_BF16)
                N.call("ns_fill_normal", dev.handle, a.ptr, N.NS_BF16, C.c_int64(m * k_), 1, 0.0, 1.0)
                y = dev.empty(m * n_, N.NS_BF16)
                us = timed_graph(lambda i: N.call("ns_matmul_bf16", dev.handle, a.ptr, ws[i % copies].ptr, y.ptr, 1, m, n_, k_, 0, 0, 0, 0, N.EPI_NONE,
                                                  N.NS_BF16))
                nbytes = 2 * (m * k_ + k_ * n_ + m * n_)
            gbs = nbytes / (us * 1e-6) / 1e9
            net = nbytes / (max(us - floor_us, 1e-3) * 1e-6) / 1e9
            rows.append({"kind": kind, "M": m, "N": n_, "K": k_, "us": us, "algorithmic_bytes": nbytes, "gbs": gbs, "hbm_frac": gbs / peaks["hbm"],
                         "hbm_time_us": nbytes / peaks["hbm"] / 1e3, "hbm_frac_net_of_launch_floor": net / peaks["hbm"], "weight_copies": copies})
            for w in ws:
                w.release()
        print(json.dumps({"case": spec, "ok": True, "launch_floor_us": floor_us, "hbm_peak_gbs": peaks["hbm"], "shapes": rows}))
        return
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
    elif name == "prefill_parts":
        # One decoder layer of the prompt read (batch 64 x 512 positions = 32768 rows, d 2048, 16 heads, ff 8192), operator by
        # operator, each timed alone over 10 launches: where a layer's time goes, and what rate each row kernel reaches.
        from nn_b200.gpt import GptConfig, GptW8A8
        peaks = measured_peaks()
        g = GPT
        B, S = g["batch"], g["prompt"]
        cfg = GptConfig(vocab=g["vocab"], dim=g["dim"], heads=g["heads"], layers=1, ff_dim=g["ff_dim"], context=S + 8)
        model = GptW8A8(dev, cfg, SyntheticGptWeights(cfg, g["seed"]), B, max_prefill=S)
        model.prefill(gpt_prompt(cfg, B, S, g["seed"]))       # fills every buffer with real activations
        dev.synchronize()
        h, D, FF, dh, m = dev.handle, cfg.dim, cfg.ff_dim, cfg.head_dim, B * S
        L, cache = model.layers[0], model.caches[0]
        x_in, x_out = model.x
        eps, scale = C.c_float(cfg.eps), C.c_float(1.0 / np.sqrt(dh))
        q, k, v = model.qkv.ptr, model.qkv.ptr + 2 * D, model.qkv.ptr + 4 * D
        st_in, st_out = (C.c_int64 * 3)(S * 3 * D, dh, 3 * D), (C.c_int64 * 3)(S * D, dh, D)
        zero_pos = dev.zeros(B, N.NS_I32)
        ops = [
            ("layernorm -> int8 [m, 2048]", 3 * m * D, 0,
             lambda: N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, L["ln1"][0].ptr, L["ln1"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, model.hq.ptr, model.hq_scale.ptr)),
            ("qkv product [m, 2048] x [2048, 6144]", m * D + 6 * m * D, 2 * m * D * 3 * D,
             lambda: L["qkv"].forward(model.hq.ptr, model.hq_scale.ptr, m, N.EPI_BIAS, N.NS_BF16, model.qkv.ptr)),
            ("key / value append", 8 * m * D, 0,
             lambda: N.call("ns_kv_append", h, cache, C.c_uint64(k), C.c_uint64(v), C.c_int64(3 * D), model.page_table.ptr, model.max_pages, zero_pos.ptr, B, S)),
            ("causal attention", 8 * m * D, 2 * 2 * B * cfg.heads * S * S * dh // 2,
             lambda: N.call("ns_attention_prefill", h, C.c_uint64(q), C.c_uint64(k), C.c_uint64(v), model.attn.ptr, B, cfg.heads, S, dh, st_in, st_in, st_in, st_out, scale, 1)),
            ("quantise [m, 2048]", 3 * m * D, 0,
             lambda: N.call("ns_quantize_rows_i8", h, model.attn.ptr, N.NS_BF16, C.c_int64(m), D, model.hq.ptr, model.hq_scale.ptr)),
            ("output product + residual [m, 2048] x [2048, 2048]", m * D + 4 * m * D, 2 * m * D * D,
             lambda: L["out"].forward(model.hq.ptr, model.hq_scale.ptr, m, N.EPI_BIAS_RESIDUAL, N.NS_BF16, x_out.ptr, residual=x_in.ptr)),
            ("ff1 product + GELU [m, 2048] x [2048, 8192]", m * D + 2 * m * FF, 2 * m * D * FF,
             lambda: L["ff1"].forward(model.hq.ptr, model.hq_scale.ptr, m, N.EPI_BIAS_GELU, N.NS_BF16, model.ffh.ptr)),
            ("quantise [m, 8192]", 3 * m * FF, 0,
             lambda: N.call("ns_quantize_rows_i8", h, model.ffh.ptr, N.NS_BF16, C.c_int64(m), FF, model.hq.ptr, model.hq_scale.ptr)),
            ("ff2 product + residual [m, 8192] x [8192, 2048]", m * FF + 4 * m * D, 2 * m * D * FF,
             lambda: L["ff2"].forward(model.hq.ptr, model.hq_scale.ptr, m, N.EPI_BIAS_RESIDUAL, N.NS_BF16, x_out.ptr, residual=x_in.ptr)),
        ]
        e0, e1 = dev.event(), dev.event()
        rows, total = [], 0.0
        for label, nbytes, nops, fn in ops:
            for _ in range(3):
                fn()
            dev.synchronize()
            dev.record(e0)
            for _ in range(10):
                fn()
            dev.record(e1)
            dev.synchronize()
            us = dev.elapsed_ms(e0, e1) * 100.0
            total += us
            gbs = nbytes / (us * 1e-6) / 1e9
            rows.append({"op": label, "us": us, "bytes": nbytes, "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm"],
                         "tops": nops / (us * 1e-6) / 1e12 if nops else None})
        print(json.dumps({"case": spec, "ok": True, "rows": m, "layer_us": total, "hbm_peak_gbs": peaks["hbm"], "ops": rows}))
        model.close()
        return
    elif name == "gpt_decode":
        from nn_b200 import dist as nsdist
        parts = arg.split(":") + ["", "", "", "", "", ""]
        rank, world, _ = nsdist.env_rank()
        rec = run_gpt_decode(dev, rank, world, measured_peaks(), int(parts[0] or 2), int(parts[1] or 64), compare_tp1=False,
                             fused=int(parts[2]) if parts[2] else None, attn_quant=bool(int(parts[3])) if parts[3] else None,
                             batch=int(parts[4]) if parts[4] else None, unfused_rows=int(parts[5]) if parts[5] else None)
        if rank == 0:
            print(json.dumps({"case": spec, "ok": True, "gpt_decode": rec}))
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
    ap.add_argument("--no-gpt", action="store_true", help="skip the decoder's generation (the int8 product line only)")
    ap.add_argument("--short", action="store_true", help="for launch lists under a profiler: exactly --steps timed steps, no loaded phases around "
                                                         "them, no main-loop yardstick (the numbers printed are then not benchmark values)")
    ap.add_argument("--no-tp1", action="store_true", help="several GPUs: skip the one-GPU run the tokens are compared with")
    ap.add_argument("--gpt-layers", type=int, default=GPT["layers"])
    ap.add_argument("--gpt-tokens", type=int, default=GPT["new_tokens"])
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
