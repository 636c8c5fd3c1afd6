"""Decoder-only GPT on the int8 / bf16 path: the host side of the reference's generator, over the C ABI.

Mirrors ``CharGpt.Create`` / ``CharGpt.Generate`` (samples/Shared/Gpt/CharGpt.cs:107-124,161-336) and
``Sequential.ForwardCached`` / ``TransformerEncoderLayer.ForwardCached`` / ``MultiHeadAttention.ForwardCached``
(src/NeuralSharp/Layers/Sequential.cs:59-80, Layers/Attention.cs:98-118,201-211): pre-LayerNorm blocks
``x + Attn(LN(x))``, ``x + FF2(GELU(FF1(LN(x))))``, final LayerNorm, head; prefill, then one cached step per token
replayed as a CUDA graph with the position and the sampled ids living on the device (Layers/Decoding.cs:81-82,
129-155); when the context is full the last half is re-read from position 0 (CharGpt.cs:276-283).

Arithmetic (the float32-only reference has no counterpart; the CPU oracle in oracle/model.py states the same
rules): weights int8 per output channel, every Linear input quantised per row from its bf16 value, exact int32
accumulation, float dequantisation + bias (+GELU, +residual), residual stream / KV cache bf16, LayerNorm and
softmax statistics float, logits float, greedy token = first maximum.

Tensor parallelism (new; the reference is single-device): QKV and FF1 are split by columns (heads stay whole),
out-projection and FF2 by rows with a float all-reduce of the partial sums, the head by vocabulary columns with a
(value, index) merge.  One process per GPU; ``comm`` is a communicator made with ``ns_comm_init_rank``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import native as N
from .device import Device, Storage


@dataclass
class GptConfig:
    vocab: int
    dim: int
    heads: int
    layers: int
    ff_dim: int
    context: int
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads


def _bf16(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bits, round to nearest even (host-side preparation of the embedding tables)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


class _Linear:
    def __init__(self, dev: Device, w_kn: np.ndarray, bias, split: int, groups: int, rank: int, size: int, mode: int = N.NS_I8):
        w = np.ascontiguousarray(w_kn, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        h = C.c_void_p()
        N.call("ns_linear_create", dev.handle, w.shape[0], w.shape[1], mode, w.ctypes.data_as(C.POINTER(C.c_float)),
               None if b is None else b.ctypes.data_as(C.POINTER(C.c_float)), split, groups, rank, size, C.byref(h))
        self.handle, self.dev = h, dev
        k, n, bias_ptr = C.c_int(), C.c_int(), C.c_uint64()
        N.call("ns_linear_info", h, C.byref(k), C.byref(n), None, None, None, C.byref(bias_ptr))
        self.k_local, self.n_local, self.bias_ptr = k.value, n.value, bias_ptr.value

    def forward(self, x: int, x_scale: int, m: int, epilogue: int, out_dtype: int, y: int, residual: int = 0, residual_dtype: int = N.NS_BF16):
        N.call("ns_linear_forward", self.dev.handle, self.handle, C.c_uint64(x), C.c_uint64(x_scale), m, epilogue, C.c_uint64(residual),
               residual_dtype, out_dtype, C.c_uint64(y))

    def forward_partial(self, x: int, m: int):
        """The product without its epilogue: (address, splits) of the int32 partial sums in the device's scratch block."""
        ptr, splits = C.c_uint64(), C.c_int()
        N.call("ns_linear_forward_partial", self.dev.handle, self.handle, C.c_uint64(x), m, C.byref(ptr), C.byref(splits))
        return ptr.value, splits.value

    def close(self):
        if self.handle:
            N.call("ns_linear_destroy", self.handle)
            self.handle = None


# Up to this many rows a pass uses the fused row kernels (ns_finish_*): one launch less per product whose K is split.
FUSED_MAX_ROWS = 256
# A prompt of at least this many positions read from position 0 (head_dim 128) takes the flash-attention kernel, a shorter one
# the cached-attention kernel -- by the prompt's length alone, whatever the batch, so that a sequence read in a batch and the
# same sequence read alone go through the same arithmetic.
FLASH_MIN_STEPS = 128
# Up to this many rows an int8 product is ONE streaming kernel with its epilogue inside (1-8 rows: dp4a, weights read once at
# the HBM rate; 9-16 rows: weights straight into registers, mma.sync).
STREAM_MAX_ROWS = 16


class GptW8A8:
    """weights: dict of float32 arrays in the reference's layouts --
    tok [V, D], pos [context, D], lnf_g, lnf_b [D], head_w [D, V], head_b [V], and per layer i:
    ln1_g, ln1_b, qkv_w [D, 3D], qkv_b, out_w [D, D], out_b, ln2_g, ln2_b, ff1_w [D, FF], ff1_b, ff2_w [FF, D], ff2_b
    under keys f"l{i}.<name>" (Linear.Weight is [in, out], Layers/Linear.cs:25-27).  Any mapping works: every tensor
    is looked up once, layer by layer, so a caller may produce them on demand.
    """

    def __init__(self, dev: Device, cfg: GptConfig, weights: dict, batch: int, max_prefill: int, tp_rank: int = 0, tp_size: int = 1,
                 comm=None, page_size: int = 64, peer_exchange: bool = True):
        assert cfg.dim % cfg.heads == 0 and cfg.heads % tp_size == 0 and cfg.ff_dim % tp_size == 0 and cfg.vocab % tp_size == 0
        assert tp_size == 1 or comm is not None
        self.dev, self.cfg, self.batch, self.rank, self.tp, self.comm = dev, cfg, batch, tp_rank, tp_size, comm
        D, FF, V = cfg.dim, cfg.ff_dim, cfg.vocab
        self.heads_loc, self.d_loc, self.ff_loc, self.v_loc = cfg.heads // tp_size, D // tp_size, FF // tp_size, V // tp_size
        self.max_rows = batch * max(max_prefill, 1)
        col, row = N.SPLIT_COLUMN, N.SPLIT_ROW
        self.tok = dev.from_numpy(_bf16(weights["tok"]))
        self.pos_table = dev.from_numpy(_bf16(weights["pos"]))
        self.lnf = (dev.from_numpy(weights["lnf_g"].astype(np.float32)), dev.from_numpy(weights["lnf_b"].astype(np.float32)))
        self.head = _Linear(dev, weights["head_w"], weights["head_b"], col, 1, tp_rank, tp_size)
        self.layers = []
        for i in range(cfg.layers):
            w = (lambda name, i=i: weights[f"l{i}.{name}"])
            self.layers.append({
                "ln1": (dev.from_numpy(w("ln1_g").astype(np.float32)), dev.from_numpy(w("ln1_b").astype(np.float32))),
                "ln2": (dev.from_numpy(w("ln2_g").astype(np.float32)), dev.from_numpy(w("ln2_b").astype(np.float32))),
                "qkv": _Linear(dev, w("qkv_w"), w("qkv_b"), col, 3, tp_rank, tp_size),
                "out": _Linear(dev, w("out_w"), w("out_b"), row, 1, tp_rank, tp_size),
                "ff1": _Linear(dev, w("ff1_w"), w("ff1_b"), col, 1, tp_rank, tp_size),
                "ff2": _Linear(dev, w("ff2_w"), w("ff2_b"), row, 1, tp_rank, tp_size),
            })
        # paged key/value caches, one per layer, identity page table (= the reference's contiguous cache)
        self.page_size = page_size
        self.max_pages = (cfg.context + page_size - 1) // page_size
        self.page_table = dev.from_numpy(np.arange(batch * self.max_pages, dtype=np.int32))
        # the pools of every layer in ONE allocation (keys of layer 0, values of layer 0, keys of layer 1, ...), so that the
        # other ranks of a tensor-parallel run can map them and deliver prompt keys / values (batch-sharded prefill)
        self.pool_bytes = batch * self.max_pages * self.heads_loc * page_size * cfg.head_dim * 2
        self.kv_block = dev.empty(2 * cfg.layers * self.pool_bytes, N.NS_I8)
        self.caches = []
        for i in range(cfg.layers):
            h = C.c_void_p()
            N.call("ns_kv_cache_create_in", dev.handle, batch * self.max_pages, page_size, self.heads_loc, cfg.head_dim,
                   C.c_uint64(self.kv_block.ptr + 2 * i * self.pool_bytes), C.c_uint64(self.kv_block.ptr + (2 * i + 1) * self.pool_bytes), C.byref(h))
            self.caches.append(h)
        self.after_kv_append = None    # callback(layer) of the many-row pass, right after a layer's keys / values are in the cache
        self.replica = None            # a one-GPU model of batch / tp sequences for the batch-sharded prompt read
        self._peer_kv = None           # every rank's kv_block as mapped here
        self._bar = None
        # activations (sized for the longest prefill) and device-side state
        R = self.max_rows
        self.x = [dev.empty(R * D, N.NS_BF16), dev.empty(R * D, N.NS_BF16)]
        self.hq, self.hq_scale = dev.empty(R * max(D, self.ff_loc), N.NS_I8), dev.empty(R)
        self.qkv = dev.empty(R * 3 * self.d_loc, N.NS_BF16)
        self.attn = dev.empty(R * self.d_loc, N.NS_BF16)
        self.ffh = dev.empty(R * self.ff_loc, N.NS_BF16)
        self.partial = dev.empty(R * D, N.NS_F32) if tp_size > 1 else None
        # few-row passes on several GPUs exchange their partial rows through peer memory (one fused kernel per half-layer)
        self.peer = None
        self.peer_slots = None
        self._peer_all = self._peer_solo = None
        if tp_size > 1 and peer_exchange and D % 256 == 0 and D <= 8192:
            from . import dist
            self.peer = dist.make_peer_group(dev, tp_rank, tp_size, FUSED_MAX_ROWS * D * 4)
            self.peer_slots = []
            for slot in range(2):
                ptr = C.c_uint64()
                N.call("ns_peer_group_slot", self.peer, slot, C.byref(ptr))
                self.peer_slots.append(ptr.value)
            self._peer_all = (self.peer, self.peer_slots)
        self.last = dev.empty(batch * D, N.NS_BF16)
        self.logits = dev.empty(batch * self.v_loc, N.NS_F32)
        self.ids = dev.zeros(self.max_rows, N.NS_I32)          # prompt ids during prefill; ids[0:batch] = current tokens while decoding
        self.pos = dev.zeros(1, N.NS_I32)
        if tp_size > 1:
            self.am_val, self.am_idx = dev.empty(batch), dev.empty(batch, N.NS_I32)
            self.am_vals, self.am_idxs = dev.empty(batch * tp_size), dev.empty(batch * tp_size, N.NS_I32)
        self.length = 0          # host mirror of the device position (DecodingContext.Length, Layers/Decoding.cs:75)
        # few-row passes: 1 = product kernel + fused row kernel (the default: fastest, the next product's weight fetch
        # overlaps the row kernel), 2 = one launch per Linear (the row operator runs as the product kernel's second phase;
        # fewer launches, measured slower), 0 / False = one kernel per operator
        self.fused = 1
        # passes of up to this many rows take one kernel per operator instead (their products are one-launch streaming
        # kernels with the epilogue inside)
        self.unfused_rows = STREAM_MAX_ROWS
        # True: FF1's split sum + bias + GELU + quantisation as ONE row kernel (ns_finish_gelu_quant) instead of the product's own
        # second kernel + the row quantisation.  Measured on the 24-layer model, batch 64: 2.44-2.50 ms per step against 2.40-2.42
        # (64 CTAs do the GELU of 8192 columns that 512 do otherwise), so it stays off.
        self.ff1_finish = False
        # True: decode attention quantises its output rows itself (ns_attention_decode_quant: one launch less per layer).
        # Measured on the 24-layer model, batch 64: 2.49 ms per step against 2.44 with the row kernel of its own (the last
        # CTA of a row works alone while the others have left), so it stays off.
        self.attn_quant = False
        self.graph = None
        self.launches_per_step = 0

    # ------------------------------------------------------------------ one pass over `steps` new positions
    def _reduce_rows(self, lin: _Linear, m: int, x_in: Storage, x_out: Storage):
        """Row-parallel Linear + residual: fused epilogue on one GPU; partial sums, all-reduce, bias + residual on several."""
        h, D = self.dev.handle, self.cfg.dim
        if self.tp == 1:
            lin.forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_BIAS_RESIDUAL, N.NS_BF16, x_out.ptr, residual=x_in.ptr)
            self._n += 1
        else:
            lin.forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_NONE, N.NS_F32, self.partial.ptr)
            N.call("ns_allreduce", h, self.comm, C.c_uint64(self.partial.ptr), C.c_int64(m * D), N.NS_F32)
            N.call("ns_bias_residual", h, C.c_uint64(self.partial.ptr), C.c_uint64(lin.bias_ptr), C.c_uint64(x_in.ptr), N.NS_BF16,
                   C.c_int64(m), D, N.NS_BF16, C.c_uint64(x_out.ptr))
            self._n += 3

    def _forward(self, steps: int) -> None:
        """Sequential.ForwardCached for `steps` new positions of every sequence, then the greedy token of the last
        position into ids[0:batch] and position += steps -- all queued on the device's stream."""
        cfg, dev, B = self.cfg, self.dev, self.batch
        h, D, dh, dl = dev.handle, cfg.dim, cfg.head_dim, self.d_loc
        m = B * steps
        assert m <= self.max_rows and self.length + steps <= cfg.context, "DecodingContext.BeginStep: capacity exceeded"
        self._n = 0
        eps, scale = C.c_float(cfg.eps), C.c_float(1.0 / np.sqrt(dh))
        if m <= FUSED_MAX_ROWS and self.fused == 2 and self._one_launch_ok(m):
            return self._forward_one_launch(steps)
        # (one to sixteen rows: the products are streaming kernels with their epilogues inside, one launch each, and the pass
        # with one kernel per operator is the faster one -- 1.24 against 1.38 ms per step at batch 8, 1.30 against 1.45 at 16)
        if self.tp == 1 and self.unfused_rows < m <= FUSED_MAX_ROWS and self.fused:
            return self._forward_fused(steps)
        if self.tp > 1 and m <= FUSED_MAX_ROWS and self.fused and self.peer is not None:
            return self._forward_tp_fused(steps)
        x_in, x_out = self.x
        N.call("ns_embed_pos", h, self.ids.ptr, self.tok.ptr, self.pos_table.ptr, N.NS_BF16, self.pos.ptr, B, steps, D, cfg.vocab, cfg.context,
               N.NS_BF16, x_in.ptr)
        self._n += 1
        whole_sequence = self._whole_sequence(steps)
        for li, (L, cache) in enumerate(zip(self.layers, self.caches)):
            N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, L["ln1"][0].ptr, L["ln1"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, self.hq.ptr, self.hq_scale.ptr)
            L["qkv"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_BIAS, N.NS_BF16, self.qkv.ptr)
            q, k, v = self.qkv.ptr, self.qkv.ptr + 2 * dl, self.qkv.ptr + 4 * dl
            N.call("ns_kv_append", h, cache, C.c_uint64(k), C.c_uint64(v), C.c_int64(3 * dl), self.page_table.ptr, self.max_pages, self.pos.ptr, B, steps)
            if self.after_kv_append is not None:
                self.after_kv_append(li)
            if whole_sequence:
                st_in = (C.c_int64 * 3)(steps * 3 * dl, dh, 3 * dl)
                st_out = (C.c_int64 * 3)(steps * dl, dh, dl)
                N.call("ns_attention_prefill", h, C.c_uint64(q), C.c_uint64(k), C.c_uint64(v), self.attn.ptr, B, self.heads_loc, steps, dh,
                       st_in, st_in, st_in, st_out, scale, 1)
            else:
                N.call("ns_attention_decode", h, cache, C.c_uint64(q), C.c_int64(3 * dl), self.attn.ptr, C.c_int64(dl), self.page_table.ptr,
                       self.max_pages, self.pos.ptr, B, steps, scale)
            N.call("ns_quantize_rows_i8", h, self.attn.ptr, N.NS_BF16, C.c_int64(m), dl, self.hq.ptr, self.hq_scale.ptr)
            self._n += 5
            self._reduce_rows(L["out"], m, x_in, x_out)
            x_in, x_out = x_out, x_in
            N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, L["ln2"][0].ptr, L["ln2"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, self.hq.ptr, self.hq_scale.ptr)
            L["ff1"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_BIAS_GELU, N.NS_BF16, self.ffh.ptr)
            N.call("ns_quantize_rows_i8", h, self.ffh.ptr, N.NS_BF16, C.c_int64(m), self.ff_loc, self.hq.ptr, self.hq_scale.ptr)
            self._n += 3
            self._reduce_rows(L["ff2"], m, x_in, x_out)
            x_in, x_out = x_out, x_in
        # only the last position is sampled (Sampling.cs:122); the head is computed for that position alone
        if steps == 1:
            last = x_in.ptr
        else:
            N.call("ns_d2d_2d_async", h, C.c_uint64(self.last.ptr), C.c_uint64(D * 2), C.c_uint64(x_in.ptr + (steps - 1) * D * 2),
                   C.c_uint64(steps * D * 2), C.c_uint64(D * 2), C.c_uint64(B))
            last = self.last.ptr
        N.call("ns_layernorm", h, C.c_uint64(last), N.NS_BF16, self.lnf[0].ptr, self.lnf[1].ptr, C.c_int64(B), D, eps, N.NS_I8, self.hq.ptr, self.hq_scale.ptr)
        self.head.forward(self.hq.ptr, self.hq_scale.ptr, B, N.EPI_BIAS, N.NS_F32, self.logits.ptr)
        if self.tp == 1:
            N.call("ns_argmax_i32", h, self.logits.ptr, B, cfg.vocab, C.c_int64(cfg.vocab), self.ids.ptr)
            self._n += 3
        else:
            N.call("ns_argmax_partial", h, self.logits.ptr, B, self.v_loc, C.c_int64(self.v_loc), self.rank * self.v_loc, self.am_val.ptr, self.am_idx.ptr)
            N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_val.ptr), C.c_uint64(self.am_vals.ptr), C.c_int64(B), N.NS_F32)
            N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_idx.ptr), C.c_uint64(self.am_idxs.ptr), C.c_int64(B), N.NS_I32)
            N.call("ns_argmax_merge", h, self.am_vals.ptr, self.am_idxs.ptr, self.tp, B, self.ids.ptr)
            self._n += 6
        N.call("ns_add_i32", h, self.pos.ptr, steps)
        self._n += 1
        self.x = [x_in, x_out]

    def _whole_sequence(self, steps: int) -> bool:
        return steps >= FLASH_MIN_STEPS and self.length == 0 and self.cfg.head_dim == 128

    def _attention_rows(self, cache, B: int, steps: int, scale) -> None:
        """Cached attention of the new positions, output rows quantised for the output projection (hq, hq_scale)."""
        h, dl, m = self.dev.handle, self.d_loc, B * steps
        if self._whole_sequence(steps):
            dh = self.cfg.head_dim
            q, k, v = self.qkv.ptr, self.qkv.ptr + 2 * dl, self.qkv.ptr + 4 * dl
            st_in = (C.c_int64 * 3)(steps * 3 * dl, dh, 3 * dl)
            st_out = (C.c_int64 * 3)(steps * dl, dh, dl)
            N.call("ns_attention_prefill", h, C.c_uint64(q), C.c_uint64(k), C.c_uint64(v), self.attn.ptr, B, self.heads_loc, steps, dh,
                   st_in, st_in, st_in, st_out, scale, 1)
            N.call("ns_quantize_rows_i8", h, self.attn.ptr, N.NS_BF16, C.c_int64(m), dl, self.hq.ptr, self.hq_scale.ptr)
        elif self.attn_quant and m <= 4000:
            N.call("ns_attention_decode_quant", h, cache, C.c_uint64(self.qkv.ptr), C.c_int64(3 * dl), self.attn.ptr, C.c_int64(dl), self.page_table.ptr,
                   self.max_pages, self.pos.ptr, B, steps, scale, self.hq.ptr, self.hq_scale.ptr)
            self._n -= 1
        else:
            N.call("ns_attention_decode", h, cache, C.c_uint64(self.qkv.ptr), C.c_int64(3 * dl), self.attn.ptr, C.c_int64(dl), self.page_table.ptr,
                   self.max_pages, self.pos.ptr, B, steps, scale)
            N.call("ns_quantize_rows_i8", h, self.attn.ptr, N.NS_BF16, C.c_int64(m), dl, self.hq.ptr, self.hq_scale.ptr)

    def _forward_fused(self, steps: int) -> None:
        """The same pass for few rows (a decoding step) with the products' epilogues moved into the row kernels that
        follow them: per layer QKV product, dequantise + bias + KV append, attention, quantise, out product, dequantise +
        bias + residual + LayerNorm + quantise, FF1 (bias + GELU epilogue), quantise, FF2 product, dequantise + bias +
        residual + the NEXT LayerNorm + quantise: 10 launches (FF1 may add a split-K reduction of its own)."""
        cfg, dev, B = self.cfg, self.dev, self.batch
        h, D, dh, dl = dev.handle, cfg.dim, cfg.head_dim, self.d_loc
        m = B * steps
        eps, scale = C.c_float(cfg.eps), C.c_float(1.0 / np.sqrt(dh))
        x_in, x_out = self.x
        N.call("ns_embed_pos", h, self.ids.ptr, self.tok.ptr, self.pos_table.ptr, N.NS_BF16, self.pos.ptr, B, steps, D, cfg.vocab, cfg.context,
               N.NS_BF16, x_in.ptr)
        first = self.layers[0]
        N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, first["ln1"][0].ptr, first["ln1"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, self.hq.ptr, self.hq_scale.ptr)
        self._n += 2
        head_from_last_rows = steps == 1        # the final LayerNorm can ride on the last layer's FF2 only if every row is a last row
        for i, (L, cache) in enumerate(zip(self.layers, self.caches)):
            part, sp = L["qkv"].forward_partial(self.hq.ptr, m)
            N.call("ns_finish_kv_append", h, C.c_uint64(part), sp, L["qkv"].handle, self.hq_scale.ptr, B, steps, self.qkv.ptr, cache,
                   self.page_table.ptr, self.max_pages, self.pos.ptr)
            self._attention_rows(cache, B, steps, scale)
            part, sp = L["out"].forward_partial(self.hq.ptr, m)
            N.call("ns_finish_norm_quant", h, C.c_uint64(part), sp, L["out"].handle, self.hq_scale.ptr, x_in.ptr, C.c_int64(m), x_out.ptr,
                   L["ln2"][0].ptr, L["ln2"][1].ptr, eps, self.hq.ptr, self.hq_scale.ptr)
            x_in, x_out = x_out, x_in
            if self.ff1_finish and self._row_shape_ok(self.ff_loc):
                part, sp = L["ff1"].forward_partial(self.hq.ptr, m)
                N.call("ns_finish_gelu_quant", h, C.c_uint64(part), sp, L["ff1"].handle, self.hq_scale.ptr, C.c_int64(m), self.hq.ptr, self.hq_scale.ptr)
            else:
                L["ff1"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_BIAS_GELU, N.NS_BF16, self.ffh.ptr)
                N.call("ns_quantize_rows_i8", h, self.ffh.ptr, N.NS_BF16, C.c_int64(m), self.ff_loc, self.hq.ptr, self.hq_scale.ptr)
            part, sp = L["ff2"].forward_partial(self.hq.ptr, m)
            if i + 1 < len(self.layers):
                g, bta = self.layers[i + 1]["ln1"]
            elif head_from_last_rows:
                g, bta = self.lnf
            else:
                g = bta = None
            N.call("ns_finish_norm_quant", h, C.c_uint64(part), sp, L["ff2"].handle, self.hq_scale.ptr, x_in.ptr, C.c_int64(m), x_out.ptr,
                   g.ptr if g else 0, bta.ptr if bta else 0, eps, self.hq.ptr, self.hq_scale.ptr)
            x_in, x_out = x_out, x_in
            self._n += 10
        if not head_from_last_rows:
            N.call("ns_d2d_2d_async", h, C.c_uint64(self.last.ptr), C.c_uint64(D * 2), C.c_uint64(x_in.ptr + (steps - 1) * D * 2),
                   C.c_uint64(steps * D * 2), C.c_uint64(D * 2), C.c_uint64(B))
            N.call("ns_layernorm", h, C.c_uint64(self.last.ptr), N.NS_BF16, self.lnf[0].ptr, self.lnf[1].ptr, C.c_int64(B), D, eps, N.NS_I8,
                   self.hq.ptr, self.hq_scale.ptr)
            self._n += 2
        self.head.forward(self.hq.ptr, self.hq_scale.ptr, B, N.EPI_BIAS, N.NS_F32, self.logits.ptr)
        N.call("ns_argmax_i32", h, self.logits.ptr, B, cfg.vocab, C.c_int64(cfg.vocab), self.ids.ptr)
        N.call("ns_add_i32", h, self.pos.ptr, steps)
        self._n += 3
        self.x = [x_in, x_out]

    @staticmethod
    def _row_shape_ok(cols: int) -> bool:
        """Rows the register-resident row code takes: a multiple of 256 columns, 1, 2 or 4 vectors of 8 per thread."""
        if cols <= 0 or cols % 256:
            return False
        vecs = cols // 8
        t = min(vecs, 256)
        return vecs % t == 0 and vecs // t in (1, 2, 4)

    def _one_launch_ok(self, m: int) -> bool:
        ok = self._row_shape_ok(self.cfg.dim) and self._row_shape_ok(self.ff_loc) and (self.heads_loc * self.cfg.head_dim) % 8 == 0
        if self.tp > 1:
            ok = ok and self.peer is not None and m <= self.dev.sm_count
        return ok

    def _forward_one_launch(self, steps: int) -> None:
        """The few-row pass with ONE launch per Linear: each int8 product kernel ends with the row operator that follows it
        (after a device-wide arrival counter): QKV -> dequantise + bias + KV append; attention (its last CTA per row
        quantises the row); output projection -> bias + residual + LayerNorm + quantise (on several GPUs: the exchange
        over peer memory first); FF1 -> bias + GELU + quantise; FF2 like the output projection, with the NEXT layer's
        LayerNorm.  Five launches per layer; results bit-identical to the other paths."""
        cfg, dev, B = self.cfg, self.dev, self.batch
        h, D, dh, dl = dev.handle, cfg.dim, cfg.head_dim, self.d_loc
        m = B * steps
        eps, scale = C.c_float(cfg.eps), C.c_float(1.0 / np.sqrt(dh))
        x_in, x_out = self.x
        hq, hs = self.hq.ptr, self.hq_scale.ptr
        N.call("ns_embed_pos", h, self.ids.ptr, self.tok.ptr, self.pos_table.ptr, N.NS_BF16, self.pos.ptr, B, steps, D, cfg.vocab, cfg.context,
               N.NS_BF16, x_in.ptr)
        first = self.layers[0]
        N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, first["ln1"][0].ptr, first["ln1"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, hq, hs)
        self._n += 2
        head_from_last_rows = steps == 1

        def reduce_norm(lin, slot, g, bta):
            gp, bp = (g.ptr, bta.ptr) if g else (0, 0)
            qp, sp = (hq, hs) if g else (0, 0)
            if self.tp == 1:
                N.call("ns_linear_forward_norm_quant", h, lin.handle, C.c_uint64(hq), C.c_uint64(hs), x_in.ptr, C.c_int64(m), x_out.ptr, gp, bp, eps, qp, sp)
            else:
                N.call("ns_linear_forward_tp_norm_quant", h, lin.handle, self.peer, slot, C.c_uint64(hq), C.c_uint64(hs), x_in.ptr, C.c_int64(m),
                       x_out.ptr, gp, bp, eps, qp, sp)

        for i, (L, cache) in enumerate(zip(self.layers, self.caches)):
            N.call("ns_linear_forward_kv_append", h, L["qkv"].handle, C.c_uint64(hq), C.c_uint64(hs), B, steps, self.qkv.ptr, cache,
                   self.page_table.ptr, self.max_pages, self.pos.ptr)
            N.call("ns_attention_decode_quant", h, cache, C.c_uint64(self.qkv.ptr), C.c_int64(3 * dl), self.attn.ptr, C.c_int64(dl), self.page_table.ptr,
                   self.max_pages, self.pos.ptr, B, steps, scale, C.c_uint64(hq), C.c_uint64(hs))
            reduce_norm(L["out"], 0, *L["ln2"])
            x_in, x_out = x_out, x_in
            N.call("ns_linear_forward_gelu_quant", h, L["ff1"].handle, C.c_uint64(hq), C.c_uint64(hs), C.c_int64(m), C.c_uint64(hq), C.c_uint64(hs))
            if i + 1 < len(self.layers):
                g, bta = self.layers[i + 1]["ln1"]
            elif head_from_last_rows:
                g, bta = self.lnf
            else:
                g = bta = None
            reduce_norm(L["ff2"], 1, g, bta)
            x_in, x_out = x_out, x_in
            self._n += 5 + (1 if self._attention_splits(steps) > 1 else 0)
        if not head_from_last_rows:
            N.call("ns_d2d_2d_async", h, C.c_uint64(self.last.ptr), C.c_uint64(D * 2), C.c_uint64(x_in.ptr + (steps - 1) * D * 2),
                   C.c_uint64(steps * D * 2), C.c_uint64(D * 2), C.c_uint64(B))
            N.call("ns_layernorm", h, C.c_uint64(self.last.ptr), N.NS_BF16, self.lnf[0].ptr, self.lnf[1].ptr, C.c_int64(B), D, eps, N.NS_I8, hq, hs)
            self._n += 2
        self.head.forward(hq, hs, B, N.EPI_BIAS, N.NS_F32, self.logits.ptr)
        if self.tp == 1:
            N.call("ns_argmax_i32", h, self.logits.ptr, B, cfg.vocab, C.c_int64(cfg.vocab), self.ids.ptr)
            self._n += 2
        else:
            N.call("ns_argmax_partial", h, self.logits.ptr, B, self.v_loc, C.c_int64(self.v_loc), self.rank * self.v_loc, self.am_val.ptr, self.am_idx.ptr)
            N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_val.ptr), C.c_uint64(self.am_vals.ptr), C.c_int64(B), N.NS_F32)
            N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_idx.ptr), C.c_uint64(self.am_idxs.ptr), C.c_int64(B), N.NS_I32)
            N.call("ns_argmax_merge", h, self.am_vals.ptr, self.am_idxs.ptr, self.tp, B, self.ids.ptr)
            self._n += 5
        N.call("ns_add_i32", h, self.pos.ptr, steps)
        self._n += 1
        self.x = [x_in, x_out]

    def _attention_splits(self, steps: int) -> int:
        """How many ways ns_attention_decode splits the cache for this pass (a combine kernel follows when > 1): the rule of
        the library (rows under two CTAs per SM are split, each part at least 256 positions, at most 32 parts)."""
        rows = self.batch * self.heads_loc * steps
        target = 2 * self.dev.sm_count
        if rows >= target:
            return 1
        return max(1, min((target + rows - 1) // rows, max(1, (self.max_pages * self.page_size) // 256), 32))

    def _forward_tp_fused(self, steps: int) -> None:
        """The few-row pass on several GPUs: as _forward_fused, but a row-parallel product (attention output, FF2) writes
        its float partial rows into this rank's peer-memory slot and ONE kernel sums the ranks' rows, adds bias and
        residual, and normalises + quantises for the next product (ns_tp_reduce_norm_quant) -- no NCCL call inside a
        layer.  The vocabulary-split head keeps its (value, index) gather over NCCL."""
        cfg, dev, B = self.cfg, self.dev, self.batch
        h, D, dh, dl = dev.handle, cfg.dim, cfg.head_dim, self.d_loc
        m = B * steps
        eps, scale = C.c_float(cfg.eps), C.c_float(1.0 / np.sqrt(dh))
        x_in, x_out = self.x
        N.call("ns_embed_pos", h, self.ids.ptr, self.tok.ptr, self.pos_table.ptr, N.NS_BF16, self.pos.ptr, B, steps, D, cfg.vocab, cfg.context,
               N.NS_BF16, x_in.ptr)
        first = self.layers[0]
        N.call("ns_layernorm", h, x_in.ptr, N.NS_BF16, first["ln1"][0].ptr, first["ln1"][1].ptr, C.c_int64(m), D, eps, N.NS_I8, self.hq.ptr, self.hq_scale.ptr)
        self._n += 2
        head_from_last_rows = steps == 1
        for i, (L, cache) in enumerate(zip(self.layers, self.caches)):
            part, sp = L["qkv"].forward_partial(self.hq.ptr, m)
            N.call("ns_finish_kv_append", h, C.c_uint64(part), sp, L["qkv"].handle, self.hq_scale.ptr, B, steps, self.qkv.ptr, cache,
                   self.page_table.ptr, self.max_pages, self.pos.ptr)
            self._attention_rows(cache, B, steps, scale)
            L["out"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_NONE, N.NS_F32, self.peer_slots[0])
            N.call("ns_tp_reduce_norm_quant", h, self.peer, 0, C.c_uint64(L["out"].bias_ptr), x_in.ptr, C.c_int64(m), D, x_out.ptr,
                   L["ln2"][0].ptr, L["ln2"][1].ptr, eps, self.hq.ptr, self.hq_scale.ptr)
            x_in, x_out = x_out, x_in
            L["ff1"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_BIAS_GELU, N.NS_BF16, self.ffh.ptr)
            N.call("ns_quantize_rows_i8", h, self.ffh.ptr, N.NS_BF16, C.c_int64(m), self.ff_loc, self.hq.ptr, self.hq_scale.ptr)
            L["ff2"].forward(self.hq.ptr, self.hq_scale.ptr, m, N.EPI_NONE, N.NS_F32, self.peer_slots[1])
            if i + 1 < len(self.layers):
                g, bta = self.layers[i + 1]["ln1"]
            elif head_from_last_rows:
                g, bta = self.lnf
            else:
                g = bta = None
            N.call("ns_tp_reduce_norm_quant", h, self.peer, 1, C.c_uint64(L["ff2"].bias_ptr), x_in.ptr, C.c_int64(m), D, x_out.ptr,
                   g.ptr if g else 0, bta.ptr if bta else 0, eps, self.hq.ptr if g else 0, self.hq_scale.ptr if g else 0)
            x_in, x_out = x_out, x_in
            self._n += 10
        if not head_from_last_rows:
            N.call("ns_d2d_2d_async", h, C.c_uint64(self.last.ptr), C.c_uint64(D * 2), C.c_uint64(x_in.ptr + (steps - 1) * D * 2),
                   C.c_uint64(steps * D * 2), C.c_uint64(D * 2), C.c_uint64(B))
            N.call("ns_layernorm", h, C.c_uint64(self.last.ptr), N.NS_BF16, self.lnf[0].ptr, self.lnf[1].ptr, C.c_int64(B), D, eps, N.NS_I8,
                   self.hq.ptr, self.hq_scale.ptr)
            self._n += 2
        self.head.forward(self.hq.ptr, self.hq_scale.ptr, B, N.EPI_BIAS, N.NS_F32, self.logits.ptr)
        N.call("ns_argmax_partial", h, self.logits.ptr, B, self.v_loc, C.c_int64(self.v_loc), self.rank * self.v_loc, self.am_val.ptr, self.am_idx.ptr)
        N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_val.ptr), C.c_uint64(self.am_vals.ptr), C.c_int64(B), N.NS_F32)
        N.call("ns_allgather", h, self.comm, C.c_uint64(self.am_idx.ptr), C.c_uint64(self.am_idxs.ptr), C.c_int64(B), N.NS_I32)
        N.call("ns_argmax_merge", h, self.am_vals.ptr, self.am_idxs.ptr, self.tp, B, self.ids.ptr)
        N.call("ns_add_i32", h, self.pos.ptr, steps)
        self._n += 6
        self.x = [x_in, x_out]

    # ------------------------------------------------------------------ generator (CharGpt.Generate, CharGpt.cs:231-318)
    def reset(self) -> None:
        """DecodingContext.Reset (Layers/Decoding.cs:84-92): position 0; stale cache rows stay masked."""
        N.call("ns_memset32_async", self.dev.handle, C.c_uint64(self.pos.ptr), 0, C.c_uint64(1))
        self.length = 0

    def enable_batch_sharded_prefill(self, weights: dict) -> None:
        """Several GPUs: from now on the prompt is read by BATCH sharding -- this rank reads batch / tp sequences with a full
        copy of the weights and no collective (the read is compute-bound and scales with the GPUs), then delivers the keys
        and values of its sequences to the ranks that own the heads (ns_kv_scatter_heads: stores into the peers' caches
        over NVLink), and the first tokens are gathered.  Decoding stays tensor-parallel.  Costs a second copy of the int8
        weights (unsharded) and a cache for batch / tp sequences on every GPU."""
        if self.tp == 1 or self.replica is not None:
            return
        assert self.batch % self.tp == 0, "the batch must divide over the ranks"
        from . import dist
        self.replica = GptW8A8(self.dev, self.cfg, weights, self.batch // self.tp, self.max_rows // self.batch, page_size=self.page_size)
        mine = C.create_string_buffer(64)
        N.call("ns_ipc_handle", self.dev.handle, C.c_uint64(self.kv_block.ptr), mine)
        # a second device object on the same GPU: its stream carries the key/value delivery of layer l while the prompt read
        # works on layer l + 1
        from .device import Device
        self._side = Device(self.dev.ordinal)
        self._kv_events = [self.dev.event() for _ in range(self.cfg.layers)]
        self._side_done = self.dev.event()
        self._peer_kv = []
        for r, handle in enumerate(dist.all_gather_bytes(mine.raw)):
            if r == self.rank:
                self._peer_kv.append(self.kv_block.ptr)
            else:
                ptr = C.c_uint64()
                N.call("ns_ipc_open", self.dev.handle, handle, C.byref(ptr))
                self._peer_kv.append(ptr.value)

    def _prefill_batch_sharded(self, ids: np.ndarray) -> None:
        from . import dist
        rep, bl, t = self.replica, self.batch // self.tp, ids.shape[1]
        h = self.dev.handle
        # Every rank must be done with its previous step (it reads its cache) before a peer overwrites that cache: a one-word
        # all-reduce queued on the stream completes on a rank only once every rank has reached it in its own stream.
        if self._bar is None:
            self._bar = self.dev.zeros(8, N.NS_I32)
        N.call("ns_allreduce", h, self.comm, C.c_uint64(self._bar.ptr), C.c_int64(1), N.NS_I32)
        pages_used = (t + self.page_size - 1) // self.page_size
        arr = C.c_uint64 * self.tp
        side = self._side
        if bl * t > FUSED_MAX_ROWS:
            # The delivery of layer l runs on the side stream while the read computes layer l + 1: the side stream first
            # waits for the barrier above (an event on the main stream), then per layer for that layer's keys / values.
            self.dev.record(self._side_done)
            side.wait_event(self._side_done)

            def deliver(layer: int) -> None:
                self.dev.record(self._kv_events[layer])
                side.wait_event(self._kv_events[layer])
                dk = arr(*[p + 2 * layer * self.pool_bytes for p in self._peer_kv])
                dv = arr(*[p + (2 * layer + 1) * self.pool_bytes for p in self._peer_kv])
                N.call("ns_kv_scatter_heads", side.handle, rep.caches[layer], rep.page_table.ptr, rep.max_pages, bl, self.rank * bl, pages_used, dk, dv,
                       self.tp, self.heads_loc, self.batch * self.max_pages, self.page_table.ptr, self.max_pages, 1, C.c_uint64(0), C.c_uint64(0))

            rep.after_kv_append = deliver
            try:
                rep.prefill(ids[self.rank * bl:(self.rank + 1) * bl])
            finally:
                rep.after_kv_append = None
            side.record(self._side_done)
            self.dev.wait_event(self._side_done)
        else:
            # a short re-read goes through the few-row pass: deliver all layers afterwards, in one launch (both models keep
            # [layer][keys, values] pools in one allocation)
            rep.prefill(ids[self.rank * bl:(self.rank + 1) * bl])
            dk = arr(*self._peer_kv)
            dv = arr(*[p + self.pool_bytes for p in self._peer_kv])
            N.call("ns_kv_scatter_heads", h, rep.caches[0], rep.page_table.ptr, rep.max_pages, bl, self.rank * bl, pages_used, dk, dv, self.tp,
                   self.heads_loc, self.batch * self.max_pages, self.page_table.ptr, self.max_pages, self.cfg.layers, C.c_uint64(2 * rep.pool_bytes),
                   C.c_uint64(2 * self.pool_bytes))
        # the first tokens of all sequences; a rank's share leaves only after its stores above are complete (stream order), and
        # the gather completes only when every rank has contributed: after it, every cache holds every sequence's prompt
        N.call("ns_allgather", h, self.comm, C.c_uint64(rep.ids.ptr), C.c_uint64(self.ids.ptr), C.c_int64(bl), N.NS_I32)
        N.call("ns_memset32_async", h, C.c_uint64(self.pos.ptr), t, C.c_uint64(1))
        self.length = t

    def prefill(self, ids: np.ndarray) -> None:
        """ids [batch, t]: reads t positions from position 0 and samples the next token into ids[0:batch]."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        b, t = ids.shape
        assert b == self.batch
        if self.replica is not None:
            return self._prefill_batch_sharded(ids)
        self.reset()
        N.call("ns_h2d", self.dev.handle, C.c_uint64(self.ids.ptr), ids.ctypes.data_as(C.c_void_p), C.c_uint64(ids.nbytes))
        self._forward(t)
        self.length = t

    def step(self, use_graph: bool = True) -> None:
        """One cached decoding step for every sequence; the first call records it as a CUDA graph
        (DecodingContext.CaptureStep / ReplayStep, Layers/Decoding.cs:129-155)."""
        assert self.length + 1 <= self.cfg.context, "context is full: re-read the window first"
        if not use_graph:
            self._forward(1)
        else:
            if self.graph is None:
                self._forward(1)               # un-captured once: sizes scratch memory, sets kernel attributes
                self.length += 1
                self.launches_per_step = self._n
                self.dev.capture_begin()
                try:
                    self._forward(1)
                except Exception:
                    N.call("ns_capture_abort", self.dev.handle)
                    raise
                self.graph = self.dev.capture_end()
                return                          # the captured pass did not execute; the un-captured one was this step
            self.dev.graph_launch(self.graph)
        self.length += 1

    def set_local_exchange(self, local: bool) -> None:
        """Measurement aid for several GPUs: with local=True the exchange kernel of the few-row pass runs in its
        single-rank form (this rank's own partial rows only: no flag traffic, no peer loads), so the step's time without
        the cross-GPU exchange can be measured.  The results are then NOT the model's.  The recorded step is dropped."""
        if self._peer_all is None:
            return
        if local and self._peer_solo is None:
            solo = C.c_void_p()
            N.call("ns_peer_group_create", self.dev.handle, 0, 1, C.c_uint64(FUSED_MAX_ROWS * self.cfg.dim * 4), C.byref(solo))
            slots = []
            for slot in range(2):
                ptr = C.c_uint64()
                N.call("ns_peer_group_slot", solo, slot, C.byref(ptr))
                slots.append(ptr.value)
            self._peer_solo = (solo, slots)
        self.peer, self.peer_slots = self._peer_solo if local else self._peer_all
        if self.graph is not None:
            self.dev.synchronize()
            self.dev.graph_destroy(self.graph)
            self.graph = None

    def read_ids(self) -> np.ndarray:
        return self.ids.download(count=self.batch).copy()

    def read_logits(self) -> np.ndarray:
        return self.logits.download((self.batch, self.v_loc))

    def generate(self, prompt: np.ndarray, n_new: int, use_graph: bool = True, marks: dict | None = None,
                 mark_every: int = 32) -> tuple[np.ndarray, int]:
        """Greedy decoding of n_new tokens per sequence; returns (tokens [batch, n_new], context resets).
        marks: when a dict is given, device events are recorded into it on the device's stream -- "start" (before the
        prompt is read), "prefill_end" (the first token is on the device), "steps" = [(tokens produced so far, event), ...]
        every mark_every decoding steps and after the last one -- for timing a generation from outside."""
        cfg, B = self.cfg, self.batch

        def mark(name=None, count=None):
            if marks is None:
                return
            e = self.dev.event()
            self.dev.record(e)
            if name is not None:
                marks[name] = e
            else:
                marks.setdefault("steps", []).append((count, e))

        history = [list(map(int, row)) for row in np.asarray(prompt)]
        hist_dev = self.dev.empty(B * max(n_new, 1), N.NS_I32)
        pending = 0            # tokens sampled on the device and not yet fetched
        out: list[list[int]] = [[] for _ in range(B)]
        resets = 0

        def flush():
            nonlocal pending
            if pending:
                got = hist_dev.download((pending, B), count=pending * B)
                for row in got:
                    for b in range(B):
                        history[b].append(int(row[b])); out[b].append(int(row[b]))
                pending = 0

        def keep_token():
            nonlocal pending
            N.call("ns_d2d_async", self.dev.handle, C.c_uint64(hist_dev.ptr + pending * B * 4), C.c_uint64(self.ids.ptr), C.c_uint64(B * 4))
            pending += 1

        def window(keep):
            return np.array([h[-keep:] for h in history], dtype=np.int32)

        mark("start")
        self.prefill(window(min(len(history[0]), cfg.context - 1)))
        keep_token()
        mark("prefill_end")
        produced = 1
        while produced < n_new:
            if self.length >= cfg.context:
                flush()
                self.prefill(window(cfg.context // 2))     # window full: re-read the last half from position 0
                keep_token()
                resets += 1
                produced += 1
                continue
            self.step(use_graph)
            keep_token()
            produced += 1
            if (produced - 1) % mark_every == 0 or produced == n_new:
                mark(count=produced)
        flush()
        self.dev.synchronize()
        return np.array(out, dtype=np.int32)[:, :n_new], resets

    def close(self) -> None:
        if self.graph is not None:
            self.dev.graph_destroy(self.graph)
            self.graph = None
        if self._peer_all is not None:
            # no rank may unmap its block while a peer's kernel can still read it
            from . import dist
            self.dev.synchronize()
            dist.barrier()
            N.call("ns_peer_group_destroy", self._peer_all[0])
            if self._peer_solo is not None:
                N.call("ns_peer_group_destroy", self._peer_solo[0])
            self.peer = self._peer_all = self._peer_solo = None
        if self._peer_kv is not None:
            from . import dist
            self.dev.synchronize()
            dist.barrier()             # no peer may still be storing into this rank's cache, nor this rank into a peer's
            for r, ptr in enumerate(self._peer_kv):
                if r != self.rank:
                    N.call("ns_ipc_close", self.dev.handle, C.c_uint64(ptr))
            self._peer_kv = None
            dist.barrier()
        if self.replica is not None:
            self.replica.close()
            self.replica = None
            self._side.synchronize()
            self._side.close()
        for c in self.caches:
            N.call("ns_kv_cache_destroy", c)
        self.caches = []
        self.kv_block.release()
        for L in self.layers:
            for k in ("qkv", "out", "ff1", "ff2"):
                L[k].close()
        self.head.close()
