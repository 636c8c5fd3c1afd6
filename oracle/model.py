"""CPU oracle of the decoder (test infrastructure only; never imported by nn_b200).

Two decoders, both wired as the reference wires them (Sequential.ForwardCached, src/NeuralSharp/Layers/
Sequential.cs:59-80; TransformerEncoderLayer.ForwardCached and MultiHeadAttention.ForwardCached,
Layers/Attention.cs:98-118,201-211; CharGpt.Create, samples/Shared/Gpt/CharGpt.cs:107-124) and driven by the
reference's generate loop with its context reset (CharGpt.cs:261-308):

  F32Decoder   the reference's own arithmetic: float32 everywhere, every operator is the oracle's restatement
               of the CPU backend (oracle/ns_oracle.c).
  W8A8Decoder  the int8 / bf16 rules the float32-only reference does not have (parity unpinned by the
               reference): int8 weights per output channel, inputs of every Linear quantised per row from their
               bf16 value, exact int32 accumulation, float dequantisation + bias (+GELU, +residual), bf16 residual
               stream and key/value cache, float LayerNorm/softmax statistics, float logits.  `tp` > 1 restates
               the tensor-parallel split: column shards for QKV / FF1 / head, row shards with per-shard input
               quantisation for out-projection / FF2, partial sums added in rank order in float.
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc


def make_weights(cfg, seed: int, std: float = 0.02, sinusoid: bool = False) -> dict:
    """Synthetic weights N(0, std) from the counter-based generator; LayerNorm gamma 1 / beta 0 and zero biases
    as the reference initialises them (Layers/Linear.cs:27, Layers/Normalization.cs) unless bias_std is wanted."""
    D, FF, V = cfg.dim, cfg.ff_dim, cfg.vocab
    w, s = {}, [seed * 1000]

    def nrm(*shape, scale=std):
        s[0] += 1
        return orc.normal(shape, s[0], scale)

    w["tok"] = nrm(V, D)
    w["pos"] = orc.sinusoid_table(cfg.context, D) if sinusoid else nrm(cfg.context, D)
    for i in range(cfg.layers):
        p = f"l{i}."
        w[p + "ln1_g"], w[p + "ln1_b"] = 1.0 + nrm(D, scale=0.05), nrm(D, scale=0.02)
        w[p + "ln2_g"], w[p + "ln2_b"] = 1.0 + nrm(D, scale=0.05), nrm(D, scale=0.02)
        w[p + "qkv_w"], w[p + "qkv_b"] = nrm(D, 3 * D), nrm(3 * D, scale=0.01)
        w[p + "out_w"], w[p + "out_b"] = nrm(D, D), nrm(D, scale=0.01)
        w[p + "ff1_w"], w[p + "ff1_b"] = nrm(D, FF), nrm(FF, scale=0.01)
        w[p + "ff2_w"], w[p + "ff2_b"] = nrm(FF, D), nrm(D, scale=0.01)
    w["lnf_g"], w["lnf_b"] = 1.0 + nrm(D, scale=0.05), nrm(D, scale=0.02)
    w["head_w"], w["head_b"] = nrm(D, V), nrm(V, scale=0.01)
    return w


class _Generator:
    """The reference's generate loop (CharGpt.cs:261-308): prefill min(len, context-1) tokens, one cached step per
    token, and when the window is full re-read the last context/2 tokens from position 0."""

    def generate(self, prompt, n_new: int, sampler=None):
        """``sampler``: an oracle.sampler.TokenSampler replacing the greedy choice (CharGpt.cs:283-300)."""
        cfg = self.cfg
        history = [list(map(int, row)) for row in np.asarray(prompt)]
        out = [[] for _ in history]
        self.logit_trace = []
        resets = 0

        def window(keep):
            return np.array([h[-keep:] for h in history], dtype=np.int64)

        def take(logits):
            ids = orc.argmax(logits).astype(np.int64) if sampler is None else sampler.sample(logits)
            self.logit_trace.append(logits.copy())
            for b, t in enumerate(ids):
                history[b].append(int(t)); out[b].append(int(t))
            return ids

        self.reset()
        ids = take(self.forward(window(min(len(history[0]), cfg.context - 1))))
        produced = 1
        while produced < n_new:
            if self.length >= cfg.context:
                self.reset()
                ids = take(self.forward(window(cfg.context // 2)))
                resets += 1
            else:
                ids = take(self.forward(ids[:, None]))
            produced += 1
        return np.array(out)[:, :n_new], resets


class F32Decoder(_Generator):
    def __init__(self, cfg, weights: dict, batch: int):
        self.cfg, self.w, self.batch = cfg, weights, batch
        H, dh = cfg.heads, cfg.head_dim
        self.k = [np.zeros((batch * H, cfg.context, dh), np.float32) for _ in range(cfg.layers)]
        self.v = [np.zeros((batch * H, cfg.context, dh), np.float32) for _ in range(cfg.layers)]
        self.length = 0

    def reset(self):
        self.length = 0

    def _split_heads(self, qkv, part, B, t):
        cfg = self.cfg
        D, H, dh = cfg.dim, cfg.heads, cfg.head_dim
        return np.ascontiguousarray(qkv[:, part * D:(part + 1) * D].reshape(B, t, H, dh).transpose(0, 2, 1, 3).reshape(B * H, t, dh))

    def forward(self, ids) -> np.ndarray:
        """ids [B, t] -> logits [B, V] of the last position (float32, reference operator order)."""
        cfg, w = self.cfg, self.w
        B, t = ids.shape
        D, H, dh, cap = cfg.dim, cfg.heads, cfg.head_dim, cfg.context
        pos = float(self.length)
        x = orc.gather(w["tok"], ids.reshape(-1).astype(np.float32)) + orc.gather(w["pos"], np.tile(np.arange(t) + pos, B).astype(np.float32))
        mask = orc.decoder_mask(pos, t, cap)
        scale = np.float32(1.0) / np.float32(np.sqrt(np.float32(dh)))
        for i in range(cfg.layers):
            p = f"l{i}."
            h = orc.layernorm_fused(x, w[p + "ln1_g"], w[p + "ln1_b"], cfg.eps)
            qkv = orc.linear_f32(h, w[p + "qkv_w"], w[p + "qkv_b"])
            q = self._split_heads(qkv, 0, B, t)
            orc.kv_write(self._split_heads(qkv, 1, B, t), self.k[i], pos)
            orc.kv_write(self._split_heads(qkv, 2, B, t), self.v[i], pos)
            raw = orc.matmul_f32(q, self.k[i], B * H, t, cap, dh, transB=True)
            weights = orc.scale_mask_softmax(raw.reshape(B * H * t, cap), mask, float(scale)).reshape(B * H, t, cap)
            o = orc.matmul_f32(weights, self.v[i], B * H, t, dh, cap)
            o = np.ascontiguousarray(o.reshape(B, H, t, dh).transpose(0, 2, 1, 3).reshape(B * t, D))
            x = x + orc.linear_f32(o, w[p + "out_w"], w[p + "out_b"])
            h2 = orc.layernorm_fused(x, w[p + "ln2_g"], w[p + "ln2_b"], cfg.eps)
            hidden = orc.bias_gelu(orc.matmul_f32(h2, w[p + "ff1_w"], 1, B * t, cfg.ff_dim, D).reshape(B * t, cfg.ff_dim), w[p + "ff1_b"])
            x = x + orc.linear_f32(hidden, w[p + "ff2_w"], w[p + "ff2_b"])
        xf = orc.layernorm_fused(x, w["lnf_g"], w["lnf_b"], cfg.eps)
        logits = orc.linear_f32(xf, w["head_w"], w["head_b"]).reshape(B, t, cfg.vocab)
        self.length += t
        return np.ascontiguousarray(logits[:, -1])


def _q_linear(x_bits, w_kn, bias, act=0, residual=None, tp=1, split="col", groups=1):
    """One W8A8 Linear on bf16 input bits [M, K]: returns float32 [M, N].  Column shards are independent output
    slices (identical to the unsplit result); row shards quantise their K-slice separately and their float
    partial sums are added in rank order, bias and residual once at the end."""
    M, K = x_bits.shape
    N = w_kn.shape[1]
    if split == "row" and tp > 1:
        ks = K // tp
        total = np.zeros((M, N), np.float32)
        for r in range(tp):
            xq, xs = orc.quantize_rows_i8(np.ascontiguousarray(x_bits[:, r * ks:(r + 1) * ks]))
            wq, ws = orc.quantize_rows_i8(np.ascontiguousarray(w_kn[r * ks:(r + 1) * ks].T))
            total = total + orc.dequant_epilogue(orc.qmatmul_i8_acc(xq, wq), xs, ws)
        y = total + bias[None, :].astype(np.float32)
        if residual is not None:
            y = y + residual
        return y.astype(np.float32)
    xq, xs = orc.quantize_rows_i8(x_bits)
    wq, ws = orc.quantize_rows_i8(np.ascontiguousarray(w_kn.T))
    return orc.dequant_epilogue(orc.qmatmul_i8_acc(xq, wq), xs, ws, bias, residual=residual, act=act)


class W8A8Decoder(_Generator):
    def __init__(self, cfg, weights: dict, batch: int, tp: int = 1):
        self.cfg, self.w, self.batch, self.tp = cfg, weights, batch, tp
        H, dh = cfg.heads, cfg.head_dim
        self.k = [np.zeros((batch, H, cfg.context, dh), np.float32) for _ in range(cfg.layers)]
        self.v = [np.zeros((batch, H, cfg.context, dh), np.float32) for _ in range(cfg.layers)]
        self.tok, self.pos = orc.bf16_round_trip(weights["tok"]), orc.bf16_round_trip(weights["pos"])
        self.length = 0

    def reset(self):
        self.length = 0

    def forward(self, ids) -> np.ndarray:
        cfg, w, tp = self.cfg, self.w, self.tp
        B, t = ids.shape
        D, H, dh = cfg.dim, cfg.heads, cfg.head_dim
        p0 = self.length
        scale = float(np.float32(1.0 / np.sqrt(dh)))
        x = orc.round_bf16(self.tok[ids.reshape(-1)] + np.tile(self.pos[p0:p0 + t], (B, 1)))      # bf16 bits [B*t, D]
        for i in range(cfg.layers):
            p = f"l{i}."
            xf = orc.widen_bf16(x)
            h = orc.round_bf16(orc.layernorm_fused(xf, w[p + "ln1_g"], w[p + "ln1_b"], cfg.eps))
            qkv = orc.bf16_round_trip(_q_linear(h, w[p + "qkv_w"], w[p + "qkv_b"])).reshape(B, t, 3, H, dh)
            self.k[i][:, :, p0:p0 + t] = qkv[:, :, 1].transpose(0, 2, 1, 3)
            self.v[i][:, :, p0:p0 + t] = qkv[:, :, 2].transpose(0, 2, 1, 3)
            o = np.empty((B, t, H, dh), np.float32)
            for b in range(B):
                for hh in range(H):
                    o[b, :, hh] = orc.attention_slice(np.ascontiguousarray(qkv[b, :, 0, hh]), self.k[i][b, hh, :p0 + t], self.v[i][b, hh, :p0 + t], p0, scale)
            ob = orc.round_bf16(o.reshape(B * t, D))
            x = orc.round_bf16(_q_linear(ob, w[p + "out_w"], w[p + "out_b"], residual=xf, tp=tp, split="row"))
            xf = orc.widen_bf16(x)
            h2 = orc.round_bf16(orc.layernorm_fused(xf, w[p + "ln2_g"], w[p + "ln2_b"], cfg.eps))
            hidden = orc.round_bf16(_q_linear(h2, w[p + "ff1_w"], w[p + "ff1_b"], act=1))
            x = orc.round_bf16(_q_linear(hidden, w[p + "ff2_w"], w[p + "ff2_b"], residual=xf, tp=tp, split="row"))
        last = orc.widen_bf16(x).reshape(B, t, D)[:, -1]
        hf = orc.round_bf16(orc.layernorm_fused(np.ascontiguousarray(last), w["lnf_g"], w["lnf_b"], cfg.eps))
        self.length += t
        return _q_linear(hf, w["head_w"], w["head_b"])
