"""The reference's float32 decoder, operator for operator, on ``NsB200Backend``.

This is the call sequence ``Sequential.ForwardCached`` issues for one cached step (src/NeuralSharp/Layers/
Sequential.cs:59-80): Embedding (gather), PositionalEncoding.ForwardCached (gather + add), per layer LayerNorm
(fused), the QKV Linear (product + AddRowVector), head split (Copy2D + Permute), KeyValueWrite, Q.K^T over the whole
cache capacity, ScaleMaskSoftmax with the decoder mask, P.V, head merge (Permute), output Linear, residual Add,
LayerNorm, product + BiasGelu, Linear, residual Add; then the final LayerNorm, the head and the greedy ArgMax of the
last position.  Ids, the position and the sampled token are float-encoded values in device memory, as in the
reference (Layers/Decoding.cs:69,81-82), so one recorded graph serves every position.

It exists to show the operator surface is a drop-in (same results as the CPU backend on the same weights) and to run
benchmark configuration 1; the fast path for large models is ``nn_b200.gpt.GptW8A8``.
"""
from __future__ import annotations

import numpy as np

from .backend import NsB200Backend
from .device import Device
from .gpt import GptConfig


class GptF32:
    def __init__(self, dev: Device, cfg: GptConfig, weights: dict, batch: int, max_steps: int):
        self.dev, self.cfg, self.batch, self.max_steps = dev, cfg, batch, max_steps
        self.be = be = NsB200Backend(dev)
        D, H, dh, FF, V, cap = cfg.dim, cfg.heads, cfg.head_dim, cfg.ff_dim, cfg.vocab, cfg.context
        up = lambda a: dev.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
        self.w = {k: up(v) for k, v in weights.items()}
        R = batch * max_steps
        a = be.Allocate
        self.ids = a(R, True)                       # float-encoded token ids [batch, steps]
        self.position = a(1, True)                  # DecodingContext.Position
        self.positions = a(max_steps, True)
        self.iota = up(np.arange(max_steps, dtype=np.float32))
        self.mask = a(max_steps * cap)
        self.x, self.x2, self.h = a(R * D), a(R * D), a(R * D)
        self.pe = a(R * D)
        self.qkv = a(R * 3 * D)
        self.part, self.q, self.kn, self.vn = a(R * D), a(R * D), a(R * D), a(R * D)
        self.scores = a(batch * H * max_steps * cap)
        self.probs = a(batch * H * max_steps * cap)
        self.ctx, self.merged = a(R * D), a(R * D)
        self.proj = a(R * D)
        self.ff = a(R * FF)
        self.ffa = a(R * FF)
        self.logits = a(R * V)
        self.keys = [a(batch * H * cap * dh, True) for _ in range(cfg.layers)]     # KeyValueCache: zero-initialised
        self.values = [a(batch * H * cap * dh, True) for _ in range(cfg.layers)]
        self.next_ids = a(batch, True)
        self.length = 0
        self.graph = None
        self.sampler = None                         # a TokenSampler replaces the greedy choice (CharGpt.cs:283-300)

    def set_sampler(self, sampler) -> None:
        """Sample with ``sampler`` (nn_b200.sampling.TokenSampler for this batch and vocabulary) instead of greedily.
        A recorded step is dropped: the sampler's kernels become part of the next recording."""
        self.sampler = sampler
        if self.graph is not None:
            self.be.DestroyGraph(self.graph)
            self.graph = None

    # Linear.ForwardCore: product, then the bias as a second kernel (Layers/Linear.cs:43-47)
    def _linear(self, x, w, b, y, m, k, n):
        self.be.MatMul(x, w, y, m, n, k, False, False, 0.0)
        self.be.AddRowVector(y, b, y, m, n)

    def _split_heads(self, part_index, dst, B, t):
        cfg, be = self.cfg, self.be
        D, H, dh = cfg.dim, cfg.heads, cfg.head_dim
        be.Copy2D(self.qkv, part_index * D, 3 * D, self.part, 0, D, B * t, D)                 # Narrow(2, part * D, D)
        be.Permute(self.part, dst, [B, H, t, dh], [t * D, dh, D, 1])                          # [B,t,H,dh] -> [B,H,t,dh]

    def forward(self, steps: int) -> None:
        cfg, be, B, w = self.cfg, self.be, self.batch, self.w
        D, H, dh, FF, V, cap = cfg.dim, cfg.heads, cfg.head_dim, cfg.ff_dim, cfg.vocab, cfg.context
        t, m = steps, B * steps
        assert self.length + t <= cap and t <= self.max_steps, "DecodingContext.BeginStep: capacity exceeded"
        # DecodingContext.BeginStep (Layers/Decoding.cs:94-118): mask and positions from the device-side position
        be.DecoderMask(self.position, self.mask, t, cap)
        be.Copy(self.iota, self.positions, t)
        be.AddBroadcastScalar(self.position, self.positions, t, 1.0)
        be.Gather(w["tok"], self.ids, self.x, m, D, V)
        be.Gather(w["pos"], self.positions, self.pe, t, D, cap)
        for b in range(B):                                                                     # broadcast add over the batch
            be.Copy2D(self.pe, 0, D, self.x, b * t * D, D, t, D, accumulate=True)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(dh)))
        x, x2 = self.x, self.x2
        for i in range(cfg.layers):
            p = f"l{i}."
            be.LayerNormFused(x, w[p + "ln1_g"], w[p + "ln1_b"], self.h, m, D, cfg.eps)
            self._linear(self.h, w[p + "qkv_w"], w[p + "qkv_b"], self.qkv, m, D, 3 * D)
            self._split_heads(0, self.q, B, t)
            self._split_heads(1, self.kn, B, t)
            self._split_heads(2, self.vn, B, t)
            be.KeyValueWrite(self.kn, self.keys[i], self.position, B * H, t, cap, dh)
            be.KeyValueWrite(self.vn, self.values[i], self.position, B * H, t, cap, dh)
            be.BatchedMatMul(self.q, self.keys[i], self.scores, B * H, t, cap, dh, False, True, 0.0)
            be.ScaleMaskSoftmax(self.scores, self.mask, self.probs, B * H * t, cap, t, scale)
            be.BatchedMatMul(self.probs, self.values[i], self.ctx, B * H, t, dh, cap, False, False, 0.0)
            be.Permute(self.ctx, self.merged, [B, t, H, dh], [H * t * dh, dh, t * dh, 1])     # [B,H,t,dh] -> [B,t,H,dh]
            self._linear(self.merged, w[p + "out_w"], w[p + "out_b"], self.proj, m, D, D)
            be.Add(x, self.proj, x2, m * D)
            x, x2 = x2, x
            be.LayerNormFused(x, w[p + "ln2_g"], w[p + "ln2_b"], self.h, m, D, cfg.eps)
            be.MatMul(self.h, w[p + "ff1_w"], self.ff, m, FF, D, False, False, 0.0)
            be.BiasGelu(self.ff, w[p + "ff1_b"], self.ffa, m * FF, FF)
            self._linear(self.ffa, w[p + "ff2_w"], w[p + "ff2_b"], self.proj, m, FF, D)
            be.Add(x, self.proj, x2, m * D)
            x, x2 = x2, x
        self.x, self.x2 = x, x2
        be.LayerNormFused(x, w["lnf_g"], w["lnf_b"], self.h, m, D, cfg.eps)
        self._linear(self.h, w["head_w"], w["head_b"], self.logits, m, D, V)
        # greedy token of the last position (TokenSampler reads row r at r * rowStride + rowOffset, Sampling.cs:122)
        if self.sampler is None:
            be.ArgMaxRows(self.logits, self.next_ids, B, V, t * V, (t - 1) * V)
        else:
            self.sampler.Sample(self.logits, t)
            be.Copy(self.sampler.Ids, self.next_ids, B)
        be.Affine(self.position, self.position, 1, 1.0, float(t))                             # DecodingContext.EndStep

    def reset(self) -> None:
        self.be.Fill(self.position, 1, 0.0)
        self.length = 0

    def prefill(self, ids: np.ndarray) -> None:
        B, t = ids.shape
        self.reset()
        buf = np.zeros(self.batch * self.max_steps, np.float32)
        buf[:B * t] = np.asarray(ids, dtype=np.float32).reshape(-1)
        self.be.Upload(buf, self.ids)
        self.forward(t)
        self.be.Copy(self.next_ids, self.ids, self.batch)
        self.length = t

    def step(self, use_graph: bool = True) -> None:
        be = self.be
        if use_graph and self.graph is None:
            be.BeginCapture()
            try:
                self.forward(1)
                be.Copy(self.next_ids, self.ids, self.batch)
            except Exception:
                be.AbortCapture()
                raise
            self.graph = be.EndCapture()
        if use_graph:
            be.ReplayGraph(self.graph)
        else:
            self.forward(1)
            be.Copy(self.next_ids, self.ids, self.batch)
        self.length += 1

    def last_logits(self, steps: int) -> np.ndarray:
        V = self.cfg.vocab
        return self.logits.download((self.batch, steps, V), count=self.batch * steps * V)[:, -1].copy()

    def generate(self, prompt: np.ndarray, n_new: int, use_graph: bool = True):
        """CharGpt.Generate's loop (CharGpt.cs:261-308) with greedy sampling; returns (tokens, resets, logits per step)."""
        cfg, B = self.cfg, self.batch
        history = [list(map(int, r)) for r in np.asarray(prompt)]
        out, trace, resets = [[] for _ in range(B)], [], 0

        def take(steps):
            self.dev.synchronize()
            ids = self.next_ids.download().astype(np.int64)
            trace.append(self.last_logits(steps))
            for b in range(B):
                history[b].append(int(ids[b])); out[b].append(int(ids[b]))

        def window(keep):
            return np.array([h[-keep:] for h in history], dtype=np.int64)

        keep = min(len(history[0]), cfg.context - 1)
        self.prefill(window(keep)); take(keep)
        produced = 1
        while produced < n_new:
            if self.length >= cfg.context:
                keep = cfg.context // 2
                self.prefill(window(keep)); take(keep)
                resets += 1
            else:
                self.step(use_graph); take(1)
            produced += 1
        return np.array(out)[:, :n_new], resets, trace
