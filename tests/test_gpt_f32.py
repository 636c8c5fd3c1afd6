"""The float32 decoder on the operator surface (nn_b200.gpt_f32.GptF32 over NsB200Backend) against the oracle's
float32 decoder (the reference's CPU backend restated), restating the reference's decoding tests:
CachedDecodingMatchesFull (DecodingTests.cs:69-98: TinyGpt vocab 11, dim 16, 4 heads, ffDim 32, 2 layers, ctx 12,
prefill 4 then 6 single steps == full forward, 1e-4), BatchedDecoding (:100-142, B=3 == each sequence alone),
GraphReplay (:144-189, graph == direct over 8 steps), and benchmark configuration 1 (char-level GPT: vocab 96, d_model 128,
4 layers, 4 heads, FFN 512, context 128, prompt 32, greedy 128 tokens: logits <= 1e-4, token ids equal, one context
reset at the 97th token).
"""
import numpy as np
import pytest

from nn_b200.gpt import GptConfig
from nn_b200.gpt_f32 import GptF32
from oracle import model as om

pytestmark = pytest.mark.gpu
TINY = GptConfig(vocab=11, dim=16, heads=4, layers=2, ff_dim=32, context=12)


def test_cached_decoding_matches_full(dev, orc):
    w = om.make_weights(TINY, seed=7, std=0.3, sinusoid=True)
    ids = orc.token_ids((1, 10), 70, TINY.vocab).astype(np.int64)
    m = GptF32(dev, TINY, w, 1, max_steps=10)
    # full forward over 10 positions
    m.prefill(ids)
    dev.synchronize()
    full = m.logits.download((10, TINY.vocab), count=10 * TINY.vocab).copy()
    ref = om.F32Decoder(TINY, w, 1)
    assert orc.close(ref.forward(ids), full[-1:], 1e-4)
    # prefill 4, then 6 single steps, teacher-forced with the same ids
    m.prefill(ids[:, :4])
    rows = [m.logits.download((4, TINY.vocab), count=4 * TINY.vocab).copy()]
    for s in range(4, 10):
        m.be.Upload(np.pad(ids[0, s:s + 1].astype(np.float32), (0, m.ids.count - 1)), m.ids)
        m.step(use_graph=False)
        dev.synchronize()
        rows.append(m.logits.download((1, TINY.vocab), count=TINY.vocab).copy())
    assert orc.close(full, np.concatenate(rows), 1e-4)


def test_batched_decoding_and_graph_replay(dev, orc):
    w = om.make_weights(TINY, seed=8, std=0.3, sinusoid=True)
    prompts = orc.token_ids((3, 3), 71, TINY.vocab).astype(np.int64)
    together = GptF32(dev, TINY, w, 3, max_steps=6)
    tok_b, _, trace_b = together.generate(prompts, 8, use_graph=True)
    tok_d, _, trace_d = together.generate(prompts, 8, use_graph=False)
    assert np.array_equal(tok_b, tok_d)                                   # GraphReplay
    for a, b in zip(trace_b, trace_d):
        assert np.array_equal(a, b)
    for i in range(3):                                                     # BatchedDecoding
        alone = GptF32(dev, TINY, w, 1, max_steps=6)
        tok_1, _, trace_1 = alone.generate(prompts[i:i + 1], 8, use_graph=False)
        for s in range(8):
            assert orc.close(trace_1[s], trace_b[s][i:i + 1], 1e-4)
    ref = om.F32Decoder(TINY, w, 3)
    exp, _ = ref.generate(prompts, 8)
    for s in range(8):
        assert orc.close(ref.logit_trace[s], trace_b[s], 1e-4)


@pytest.mark.parametrize("sinusoid", [False, True])
def test_baseline_config_1(dev, orc, sinusoid):
    cfg = GptConfig(vocab=96, dim=128, heads=4, layers=4, ff_dim=512, context=128)
    w = om.make_weights(cfg, seed=0, std=0.02, sinusoid=sinusoid)
    for k in w:
        if k.endswith("_b") and "ln" not in k:
            w[k] = np.zeros_like(w[k])                                     # biases 0, as Linear initialises them
    prompt = orc.token_ids((1, 32), 1, cfg.vocab).astype(np.int64)
    ref = om.F32Decoder(cfg, w, 1)
    exp, exp_resets = ref.generate(prompt, 128)
    assert exp_resets == 1
    m = GptF32(dev, cfg, w, 1, max_steps=64)
    got, resets, trace = m.generate(prompt, 128, use_graph=True)
    assert resets == 1
    worst, first_div = 0.0, None
    for s in range(128):
        if first_div is None and got[0, s] != exp[0, s]:
            first_div = s
        if first_div is None or s <= first_div:                            # identical histories up to the first divergence
            worst = max(worst, orc.max_err(ref.logit_trace[s], trace[s]))
    assert worst <= 1e-4, f"max logit error {worst:.2e}"
    if first_div is not None:
        top2 = np.sort(ref.logit_trace[first_div][0])[-2:]
        assert top2[1] - top2[0] <= 2e-4 * max(1.0, abs(top2[1])), f"tokens diverge at step {first_div} without a near-tie"
