"""The int8 / bf16 decoder (nn_b200.gpt.GptW8A8) against the CPU oracle decoder (oracle/model.py) on a reduced clone
of benchmark configuration 5 (same head_dim 128 and operator sequence, fewer/narrower layers so the CPU finishes in seconds).

Protocol (greedy argmax can flip on near-ties under reordered arithmetic): teacher-forced per-step comparison of the
logits and of the argmax wherever the oracle's top-2 gap exceeds the tolerance.  Every operator is held to its own
bar in its own test (int32 accumulators bit-exact, bf16 outputs 1e-2).  End to end the integer sums are exact and the
float epilogues run in the oracle's order; what differs (softmax and LayerNorm summation order, exp2 / tanh
approximations) is far below a bf16 ulp and is absorbed by the rounding to bf16 and then to int8 that follows every
operator -- unless a value sits on a rounding boundary, which moves one quantisation step of one product input.  On the
first two configurations below no such flip occurs: the logits come out bit-identical (largest error printed by the
test: 0) and the bar is the benchmark configuration's bf16 tolerance, 1e-2 * max(1, |e|).  The third (12 sequences: the
decoding steps take the one-launch streaming products for 9 to 16 rows) does have one -- the GELU of the product epilogues
is evaluated through ex2 / rcp approximations, 1e-6 relative from the oracle's tanhf form, and 12 x 8 x 512 x 2 hidden
values give a bf16 rounding boundary a chance -- and one bf16 step of a residual-stream value near 1 (2^-7) moves a
logit by about 1e-2: that configuration is held to 2e-2.  Then a free-running generation through the
CUDA graph, which must reproduce the teacher-forced run's tokens exactly (GraphReplay, DecodingTests.cs:144-189) and
hit the context reset of CharGpt.cs:276-283.
"""
import ctypes as C

import numpy as np
import pytest

from nn_b200 import native as N
from nn_b200.gpt import GptConfig, GptW8A8
from oracle import model as om

pytestmark = pytest.mark.gpu
TOL = 1e-2


WORST = {"err": 0.0}


def _check_step(orc, exp_logits, got_logits, step, tol=TOL):
    WORST["err"] = max(WORST["err"], float(orc.max_err(exp_logits, got_logits)))
    assert orc.close(exp_logits, got_logits, tol), f"step {step}: logits differ by {orc.max_err(exp_logits, got_logits):.3e}"
    top2 = np.sort(exp_logits, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2 * tol * np.maximum(1.0, np.abs(top2[:, 1]))
    agree = orc.argmax(exp_logits) == orc.argmax(got_logits)
    assert np.all(agree | ~clear), f"step {step}: argmax differs on rows {np.where(~agree & clear)[0]}"
    return int((~clear).sum())


@pytest.mark.parametrize("batch,prompt_len,n_new,context", [(3, 20, 10, 64), (2, 10, 30, 32), (12, 8, 6, 32)])
def test_teacher_forced_and_graph(dev, orc, batch, prompt_len, n_new, context):
    cfg = GptConfig(vocab=320, dim=256, heads=2, layers=2, ff_dim=512, context=context)
    w = om.make_weights(cfg, seed=4)
    prompt = orc.token_ids((batch, prompt_len), 44, cfg.vocab).astype(np.int64)
    ref = om.W8A8Decoder(cfg, w, batch)
    exp_tokens, exp_resets = ref.generate(prompt, n_new)

    model = GptW8A8(dev, cfg, w, batch, max_prefill=max(prompt_len, context // 2))
    tol = TOL if batch < 9 else 2 * TOL
    # ---- teacher-forced, no graph: the device consumes the oracle's tokens
    history = [list(r) for r in prompt]
    near_ties, step = 0, 0
    model.prefill(np.array([h[-min(len(h), context - 1):] for h in history], dtype=np.int32))
    dev.synchronize()
    near_ties += _check_step(orc, ref.logit_trace[0], model.read_logits(), 0, tol)
    for s in range(1, n_new):
        for b in range(batch):
            history[b].append(int(exp_tokens[b, s - 1]))
        forced = np.ascontiguousarray(exp_tokens[:, s - 1], dtype=np.int32)
        if model.length >= context:
            model.prefill(np.array([h[-(context // 2):] for h in history], dtype=np.int32))
        else:
            N.call("ns_h2d", dev.handle, C.c_uint64(model.ids.ptr), forced.ctypes.data_as(C.c_void_p), C.c_uint64(forced.nbytes))
            model.step(use_graph=False)
        dev.synchronize()
        near_ties += _check_step(orc, ref.logit_trace[s], model.read_logits(), s, tol)
    # ---- free-running through the graph
    tokens, resets = model.generate(prompt, n_new, use_graph=True)
    assert resets == exp_resets
    print(f"near-ties of the oracle's two best logits: {near_ties} of {batch * n_new} rows; largest logit error so far {WORST['err']:.3e}")
    if near_ties == 0:
        assert np.array_equal(tokens, exp_tokens), f"first divergence at step {np.argwhere(tokens != exp_tokens)[:1]}"
    # graph replay == direct execution
    tokens2, _ = model.generate(prompt, n_new, use_graph=False)
    assert np.array_equal(tokens, tokens2)
    model.close()


def test_oracle_tp_split_is_consistent(orc):
    """CPU only in effect: the oracle's 2-way split differs from the unsplit decoder only through per-shard
    quantisation of row-parallel inputs (logits within 5e-2)."""
    cfg = GptConfig(vocab=64, dim=256, heads=2, layers=1, ff_dim=256, context=16)
    w = om.make_weights(cfg, seed=5)
    ids = orc.token_ids((2, 6), 45, cfg.vocab).astype(np.int64)
    a = om.W8A8Decoder(cfg, w, 2, tp=1).forward(ids)
    b = om.W8A8Decoder(cfg, w, 2, tp=2).forward(ids)
    assert orc.close(a, b, 5e-2)


def test_recorded_step_survives_a_growing_scratch_block(orc):
    """A fresh device object: the step is recorded after a short prompt, then the context fills up and the window is
    re-read with MORE rows than any pass before it, so the scratch block (split-K partial sums) has to grow while the
    recorded graph still names the old block.  The old block must stay valid for the replays that follow: tokens through
    the graph equal tokens of direct execution."""
    from nn_b200.device import Device
    fresh = Device(0)
    cfg = GptConfig(vocab=320, dim=768, heads=6, layers=2, ff_dim=1536, context=32)
    w = om.make_weights(cfg, seed=9)
    prompt = orc.token_ids((2, 10), 46, cfg.vocab).astype(np.int64)
    out = []
    for use_graph in (True, False):
        model = GptW8A8(fresh, cfg, w, 2, max_prefill=16)
        tokens, resets = model.generate(prompt, 40, use_graph=use_graph)
        assert resets >= 1
        out.append(np.asarray(tokens))
        model.close()
    assert np.array_equal(out[0], out[1])
    fresh.synchronize()
    fresh.close()


def test_many_row_prompt_read(dev, orc):
    """More than 256 rows: the pass with one kernel per operator and flash attention over whole sequences (the shape of the
    benchmark's prompt read).  The flash-attention kernel rounds the softmax weights to bf16 before the P V product and is held
    to the oracle's attention at 1e-2 in its own test; over three layers the logits are held to 5e-2 here (measured: 2.2e-2).
    The pass is reproducible bit for bit, cache included, and the tokens generated after it are the same through the graph
    and through direct launches."""
    cfg = GptConfig(vocab=320, dim=256, heads=2, layers=3, ff_dim=512, context=192)
    w = om.make_weights(cfg, seed=6)
    batch, prompt_len = 4, 130
    prompt = orc.token_ids((batch, prompt_len), 46, cfg.vocab).astype(np.int32)
    ref = om.W8A8Decoder(cfg, w, batch)
    ref.generate(prompt.astype(np.int64), 1)
    out = []
    for use_graph in (True, False):
        model = GptW8A8(dev, cfg, w, batch, max_prefill=prompt_len)
        model.prefill(prompt)
        dev.synchronize()
        logits, cache = model.read_logits().copy(), model.kv_block.download().copy()
        tokens, _ = model.generate(prompt, 6, use_graph=use_graph)
        out.append((logits, cache, tokens))
        model.close()
    err = orc.max_err(ref.logit_trace[0], out[0][0])
    print(f"many-row prompt read: largest logit error {err:.3e}")
    assert orc.close(ref.logit_trace[0], out[0][0], 5e-2), err
    assert out[0][1].any()
    assert np.array_equal(out[0][0].view(np.uint32), out[1][0].view(np.uint32))
    assert np.array_equal(out[0][1], out[1][1])
    assert np.array_equal(out[0][2], out[1][2])


@pytest.mark.parametrize("prompt_len,context", [(12, 64), (40, 64), (140, 192)])
def test_a_sequence_in_a_batch_equals_the_sequence_alone(dev, orc, prompt_len, context):
    """BatchedDecoding (DecodingTests.cs:100-142), bit for bit on the int8 decoder: 20 sequences together, three of them
    together, and single ones must produce the same greedy tokens and the same logits.  The passes differ -- 20 sequences take
    the many-row pass for the prompt and tcgen05 products with fused row kernels for the steps, few sequences the streaming
    products with one kernel per operator, their attention splits the cache over several CTAs -- but every operator is exact
    (integer sums), or sums in one fixed order (LayerNorm, the chunks of cached attention), or is chosen by the prompt's length
    alone (flash attention from 128 positions on)."""
    cfg = GptConfig(vocab=320, dim=256, heads=2, layers=2, ff_dim=512, context=context)
    w = om.make_weights(cfg, seed=8)
    B, n_new = 20, 10
    prompt = orc.token_ids((B, prompt_len), 47, cfg.vocab).astype(np.int32)

    def run(rows):
        model = GptW8A8(dev, cfg, w, len(rows), max_prefill=prompt_len)
        model.prefill(prompt[rows])
        dev.synchronize()
        logits = model.read_logits().copy()
        tokens, _ = model.generate(prompt[rows], n_new, use_graph=True)
        model.close()
        return logits, tokens

    big_logits, big_tokens = run(list(range(B)))
    for rows in ([0, 1, 2], [19], [7], [4, 5, 6, 7, 8, 9, 10, 11, 12]):
        logits, tokens = run(rows)
        assert np.array_equal(logits.view(np.uint32), big_logits[rows].view(np.uint32)), f"prompt logits of sequences {rows} depend on the batch"
        assert np.array_equal(tokens, big_tokens[rows]), f"tokens of sequences {rows} depend on the batch"
