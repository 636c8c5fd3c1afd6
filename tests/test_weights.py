"""NSW2 weight files + GptConfig JSON (Module.Save/Load, src/NeuralSharp/Layers/Module.cs:204-271;
samples/Shared/Gpt/CharGpt.cs:9-31,107-138).  The byte layout is asserted against bytes assembled here with
``struct`` from the reference's writer statements, not against this package's own writer.
"""
import json
import struct

import numpy as np
import pytest

from nn_b200.gpt import GptConfig
from nn_b200 import weights as W

TINY = GptConfig(vocab=11, dim=16, heads=4, layers=2, ff_dim=64, context=12)
VOCAB = "abcdefghij\n"


def _reference_bytes(tensors):
    """BinaryWriter: Write(uint magic); Write(int count); per tensor Write(int rank), Write(int dim)..., raw LE floats."""
    b = struct.pack("<I", 0x3257534E) + struct.pack("<i", len(tensors))
    for t in tensors:
        b += struct.pack("<i", t.ndim)
        for d in t.shape:
            b += struct.pack("<i", d)
        b += b"".join(struct.pack("<f", float(v)) for v in t.reshape(-1))
    return b


def test_nsw2_layout(tmp_path):
    rng = np.random.default_rng(0)
    tensors = [rng.standard_normal((3, 5)).astype(np.float32), rng.standard_normal((7,)).astype(np.float32),
               np.zeros((0, 4), np.float32), np.float32(2.5).reshape(())]
    p = tmp_path / "m.bin"
    W.write_nsw2(str(p), tensors)
    assert p.read_bytes() == _reference_bytes(tensors)
    assert p.read_bytes()[:4] == b"NSW2"
    back = W.read_nsw2(str(p))
    assert len(back) == 4 and all(a.shape == b.shape and np.array_equal(a, b) for a, b in zip(tensors, back))


def test_nsw2_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.bin"
    p.write_bytes(b"NSW1" + b"\0" * 12)
    with pytest.raises(W.InvalidDataError, match="is not a NeuralSharp weights file"):
        W.read_nsw2(str(p))
    good = _reference_bytes([np.ones((2, 3), np.float32)])
    p.write_bytes(good[:-4])
    with pytest.raises(W.InvalidDataError, match="truncated"):
        W.read_nsw2(str(p))
    p.write_bytes(b"")
    with pytest.raises(W.InvalidDataError):
        W.read_nsw2(str(p))


def test_char_gpt_file_order_and_config(tmp_path, orc):
    from oracle import model as om
    w = om.make_weights(TINY, seed=4, sinusoid=True)
    path = str(tmp_path / "gpt.bin")
    W.save_char_gpt(path, TINY, w, VOCAB)
    # 1 embedding + 12 per block + 2 final norm + 2 head, positional table not stored
    raw = W.read_nsw2(path)
    assert len(raw) == 1 + 12 * TINY.layers + 4
    assert [tuple(t.shape) for t in raw[:7]] == [(11, 16), (16,), (16,), (16, 48), (48,), (16, 16), (16,)]
    j = json.load(open(W.config_path(path)))
    assert j["Vocabulary"] == VOCAB and (j["Context"], j["Dim"], j["Heads"], j["Layers"]) == (12, 16, 4, 2)
    cfg, back, vocab = W.load_char_gpt(path)
    assert cfg == TINY and vocab == VOCAB
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], w[k]), k          # "pos": the recomputed table equals the oracle's, bit for bit
    # record defaults (CharGpt.cs:9): Context 64, Dim 96, Heads 4, Layers 3
    json.dump({"Vocabulary": "ab"}, open(W.config_path(path), "w"))
    cfg, _ = W.read_config(path)
    assert (cfg.vocab, cfg.context, cfg.dim, cfg.heads, cfg.layers, cfg.ff_dim) == (2, 64, 96, 4, 3, 384)


def test_char_gpt_mismatch_messages(tmp_path, orc):
    from oracle import model as om
    w = om.make_weights(TINY, seed=4, sinusoid=True)
    path = str(tmp_path / "gpt.bin")
    W.save_char_gpt(path, TINY, w, VOCAB)
    W.write_config(path, GptConfig(vocab=11, dim=16, heads=4, layers=3, ff_dim=64, context=12), VOCAB)
    with pytest.raises(W.InvalidDataError, match="The file has 29 parameter tensors but the model has 41"):
        W.load_char_gpt(path)
    W.write_config(path, GptConfig(vocab=11, dim=32, heads=4, layers=2, ff_dim=128, context=12), VOCAB)
    with pytest.raises(W.InvalidDataError, match="Shape mismatch"):
        W.load_char_gpt(path)


@pytest.mark.gpu
def test_loaded_file_runs_both_decoders(tmp_path, dev, orc):
    """A weights file + config goes through the loader into the float32 decoder and the int8 decoder and gives the
    oracle's tokens."""
    from nn_b200.gpt import GptW8A8
    from nn_b200.gpt_f32 import GptF32
    from oracle import model as om
    cfg0 = GptConfig(vocab=32, dim=64, heads=2, layers=2, ff_dim=256, context=32)
    w0 = om.make_weights(cfg0, seed=9, std=0.08, sinusoid=True)
    path = str(tmp_path / "gpt.bin")
    W.save_char_gpt(path, cfg0, w0, "".join(chr(65 + i) for i in range(32)))
    cfg, w, _ = W.load_char_gpt(path)
    prompt = orc.token_ids((2, 6), 3, cfg.vocab).astype(np.int64)
    ref = om.F32Decoder(cfg, w, 2)
    exp, _ = ref.generate(prompt, 10)
    m = GptF32(dev, cfg, w, 2, max_steps=8)
    got, _, trace = m.generate(prompt, 10, use_graph=True)
    for s in range(10):
        if not np.array_equal(got[:, :s], exp[:, :s]):
            break
        assert orc.close(ref.logit_trace[s], trace[s], 1e-4)
    q = GptW8A8(dev, cfg, w, 2, max_prefill=8)
    qref = om.W8A8Decoder(cfg, w, 2)
    qexp, _ = qref.generate(prompt, 10)
    qgot, _ = q.generate(prompt, 10)
    assert (np.asarray(qgot) == np.asarray(qexp)).mean() >= 0.8
    q.close()
