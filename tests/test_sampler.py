"""TokenSampler (SampleRows / PenalizeRows / HistoryPush), restating the reference's SamplerBehaviour and SamplerFilters
(tests/NeuralSharp.Tests/DecodingTests.cs:191-250, 265-341) with the literals held in tests/golden/kat.json.

The same checks run twice: against the CPU oracle (no GPU needed: this pins the oracle to the reference's known
answers) and against the on-device sampler, which must also agree with the oracle draw for draw up to the 0.5 % of
rows the reference itself allows between its CPU and GPU backends (sums are added in another order).
"""
import json
import os

import numpy as np
import pytest

KAT = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "kat.json")))
LOGITS = np.array(KAT["sampler_logits"]["logits"], np.float32)
V = LOGITS.size
BEH, FIL = KAT["sampler_behaviour"], KAT["sampler_filters"]
ROWS = BEH["rows"]


class _OracleSide:
    """Adapter: the oracle's sampler behind the property names of the reference class."""

    def __init__(self, rows, vocabulary, max_steps, **kw):
        from oracle.sampler import TokenSampler
        self.s = TokenSampler(rows, vocabulary, max_steps)
        names = dict(Temperature="temperature", TopK="top_k", TopP="top_p", MinP="min_p", RepeatPenalty="repeat", RepeatLastN="last_n",
                     PresencePenalty="presence", FrequencyPenalty="frequency", Seed="seed")
        for k, v in kw.items():
            setattr(self.s, names[k], v)

    def SetHistory(self, tokens):
        self.s.set_history(tokens)

    def Sample(self, logits):
        self.s.sample(logits)

    def Read(self, a, b):
        return self.s.read(a, b)


class _DeviceSide:
    def __init__(self, backend, rows, vocabulary, max_steps, **kw):
        from nn_b200.sampling import TokenSampler
        self.b = backend
        self.s = TokenSampler(backend, rows, vocabulary, max_steps)
        for k, v in kw.items():
            setattr(self.s, k, v)
        self._x = {}

    def SetHistory(self, tokens):
        self.s.SetHistory(tokens)

    def Sample(self, logits):
        key = logits.ctypes.data
        if key not in self._x:
            st = self.b.Allocate(logits.size)
            self.b.Upload(logits.reshape(-1), st)
            self._x[key] = (st, logits)
        self.s.Sample(self._x[key][0])

    def Read(self, a, b):
        n = self.s.Rows * 13
        return self.b.DownloadRange(self.s._stats, a * n, (b - a) * n).reshape(b - a, self.s.Rows, 13)


def _ids(sampler, x):
    sampler.Sample(x)
    return sampler.Read(0, 1)[0][:, 0].astype(np.int64)


def _behaviour(make):
    x = np.tile(LOGITS, (ROWS, 1))
    p = np.exp(LOGITS.astype(np.float64))
    p /= p.sum()
    plain = make(ROWS, V, 1, Temperature=1.0, Seed=BEH["seed"])
    ids = _ids(plain, x)
    freq = np.bincount(ids, minlength=V) / ROWS
    assert np.all(np.abs(freq - p) < BEH["frequency_tol"]), (freq, p)
    assert np.allclose(p, KAT["sampler_logits"]["probabilities"], atol=KAT["sampler_logits"]["tol"])
    st = plain.Read(0, 1)[0][0]
    assert abs(st[1] - p[int(st[0])]) < BEH["probability_tol"]
    assert abs(st[2] - -(p * np.log2(p)).sum()) < BEH["entropy_tol"]
    assert [int(st[3]), int(st[5]), int(st[7])] == KAT["sampler_logits"]["top_order"]
    # all five alternatives: every token once, most likely first, probabilities summing to one
    assert [int(st[3 + 2 * a]) for a in range(5)] == list(np.argsort(-p, kind="stable"))
    assert abs(sum(st[4 + 2 * a] for a in range(5)) - 1.0) < 1e-5

    top = _ids(make(ROWS, V, 1, TopK=BEH["top_k"], Seed=BEH["seed"]), x)
    assert set(top) <= set(BEH["top_k_kept"])
    assert abs((top == 0).mean() - np.e / (np.e + 1)) < BEH["frequency_tol"]
    cold = _ids(make(ROWS, V, 1, Temperature=BEH["cold_temperature"], Seed=BEH["seed"]), x)
    assert np.all(cold == BEH["cold_token"])
    again = _ids(make(ROWS, V, 1, Temperature=1.0, Seed=BEH["seed"]), x)
    assert np.array_equal(again, ids), "same seed, same samples"
    other = _ids(make(ROWS, V, 1, Temperature=1.0, Seed=BEH["seed"] + 1), x)
    assert not np.array_equal(other, ids), "another seed, other samples"
    return ids


def _filters(make):
    x = np.tile(LOGITS, (ROWS, 1))
    for case in FIL["top_p"]:
        ids = _ids(make(ROWS, V, 1, TopP=case["p"], Seed=FIL["seed"]), x)
        assert set(ids) <= set(case["kept"]) and case["must_contain"] in ids, case
    case = FIL["min_p"]
    ids = _ids(make(ROWS, V, 1, MinP=case["p"], Seed=FIL["seed"]), x)
    assert set(ids) <= set(case["kept"]) and case["must_contain"] in ids

    one = LOGITS.reshape(1, V).copy()
    pen = FIL["penalties"]
    for case in pen["cases"]:
        kw = dict(Temperature=pen["temperature"], Seed=pen["seed"])
        if "repeat" in case:
            kw["RepeatPenalty"] = case["repeat"]
        if "presence" in case:
            kw["PresencePenalty"] = case["presence"]
        if "frequency" in case:
            kw["FrequencyPenalty"] = case["frequency"]
        if "last_n" in case:
            kw["RepeatLastN"] = case["last_n"]
        s = make(1, V, 1, **kw)
        s.SetHistory(pen["history"])
        assert _ids(s, one)[0] == case["token"], case

    cyc = FIL["cycle"]
    s = make(1, V, cyc["steps"], Temperature=cyc["temperature"], FrequencyPenalty=cyc["frequency"], Seed=cyc["seed"])
    for _ in range(cyc["steps"]):
        s.Sample(one)
    assert [int(t[0][0]) for t in s.Read(0, cyc["steps"])] == cyc["sequence"]

    cr = FIL["cross"]
    s = make(ROWS, V, 1, TopP=cr["top_p"], MinP=cr["min_p"], RepeatPenalty=cr["repeat"], Seed=cr["seed"])
    s.SetHistory(cr["history"])
    return _ids(s, x)


def test_oracle_sampler_behaviour():
    _behaviour(_OracleSide)


def test_oracle_sampler_filters():
    _filters(_OracleSide)


def test_oracle_history_ring_and_penalty_window():
    """The history is a ring: with capacity 4 and 6 pushed tokens only the last four count, each distinct token once."""
    from oracle import oracle as O
    cap, v = 4, 8
    hist = np.zeros((1, cap), np.float32)
    for n, t in enumerate([1, 2, 3, 3, 5, 1]):
        O.history_push(np.array([t], np.float32), hist, n, cap)
    assert hist[0].tolist() == [5, 1, 3, 3]
    z = np.arange(v, dtype=np.float32) - 3.0            # -3 .. 4
    w = O.penalize_rows(z, hist, 6, 1, v, v, 0, cap, 64, 2.0, 0.5, 0.25)[0]
    exp = z.copy()
    for tok, cnt in ((1, 1), (3, 2), (5, 1)):             # token 2 fell out of the ring
        exp[tok] = (z[tok] / 2.0 if z[tok] > 0 else z[tok] * 2.0) - 0.5 - 0.25 * cnt
    assert np.array_equal(w, exp)
    # ids outside the vocabulary are ignored
    hist[0, 0] = 99
    assert np.isfinite(O.penalize_rows(z, hist, 6, 1, v, v, 0, cap, 64, 2.0, 0.5, 0.25)).all()


@pytest.fixture(scope="module")
def backend(dev):
    from nn_b200.backend import NsB200Backend
    return NsB200Backend(dev)


@pytest.mark.gpu
def test_device_sampler_behaviour(backend):
    got = _behaviour(lambda *a, **k: _DeviceSide(backend, *a, **k))
    exp = _behaviour(_OracleSide)
    assert (got != exp).sum() <= ROWS * BEH["max_differing_fraction"]


@pytest.mark.gpu
def test_device_sampler_filters(backend):
    got = _filters(lambda *a, **k: _DeviceSide(backend, *a, **k))
    exp = _filters(_OracleSide)
    assert (got != exp).sum() <= ROWS * BEH["max_differing_fraction"]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,vocab,steps", [(1, 1, 1), (3, 7, 1), (64, 1000, 1), (5, 50257, 2), (300, 257, 3)])
def test_device_sampler_against_oracle(backend, orc, rows, vocab, steps):
    """Ragged shapes, strided rows ([rows, steps, vocabulary], last position), all filters and penalties at once,
    several steps so that history and step counter advance on the device."""
    from nn_b200.sampling import TokenSampler
    from oracle.sampler import TokenSampler as OracleSampler
    cfg = dict(Temperature=0.8, TopK=min(40, vocab), TopP=0.92, MinP=0.01, RepeatPenalty=1.2, PresencePenalty=0.1, FrequencyPenalty=0.05,
               RepeatLastN=8, Seed=1234)
    s = TokenSampler(backend, rows, vocab, 4, historyCapacity=16)
    o = OracleSampler(rows, vocab, 4, history_capacity=16)
    for k, v in cfg.items():
        setattr(s, k, v)
    (o.temperature, o.top_k, o.top_p, o.min_p, o.repeat, o.presence, o.frequency, o.last_n, o.seed) = (
        cfg["Temperature"], cfg["TopK"], cfg["TopP"], cfg["MinP"], cfg["RepeatPenalty"], cfg["PresencePenalty"], cfg["FrequencyPenalty"],
        cfg["RepeatLastN"], cfg["Seed"])
    prompt = [t % vocab for t in (3, 1, 4, 1, 5)]
    s.SetHistory(prompt)
    o.set_history(prompt)
    differing = 0
    for it in range(4):
        x = (orc.normal((rows, steps, vocab), 77 + it) * 3.0).astype(np.float32)
        st = backend.Allocate(x.size)
        backend.Upload(x.reshape(-1), st)
        s.Sample(st, steps)
        exp_ids = o.sample(x, steps)
        got_ids = backend.Download(s.Ids).astype(np.int64)
        same = got_ids == exp_ids
        differing += int((~same).sum())
        # rows that drew the same token report the same statistics
        g = backend.DownloadRange(s._stats, it * rows * 13, rows * 13).reshape(rows, 13)
        e = o.read(it, it + 1)[0]
        assert np.allclose(g[same][:, 1:3], e[same][:, 1:3], atol=2e-4), (it, np.abs(g[same][:, 1:3] - e[same][:, 1:3]).max())
        assert np.array_equal(g[same][:, 3], e[same][:, 3]), "most likely token"
        # a differing draw desynchronises the histories: realign the device's with the oracle's
        if differing:
            backend.Upload(o.history.reshape(-1), s._history)
    assert differing <= max(1, int(4 * rows * BEH["max_differing_fraction"])), differing


@pytest.mark.gpu
def test_device_sampler_in_graph(backend, dev, orc):
    """A recorded sampling step replays with the step counter and history advancing on the device
    (DecodingTests.cs:145-189 records the reference's step the same way)."""
    from nn_b200.sampling import TokenSampler
    rows, vocab, steps = 8, 300, 6
    x = (orc.normal((rows, vocab), 5) * 2.0).astype(np.float32)
    st = backend.Allocate(x.size)
    backend.Upload(x.reshape(-1), st)

    def run(graph):
        s = TokenSampler(backend, rows, vocab, steps)
        s.Temperature, s.FrequencyPenalty, s.Seed = 0.9, 0.7, 11
        out = []
        if graph:
            s.Sample(st)                      # warm-up outside capture, then rewind
            s.Reset()
            backend.BeginCapture()
            s.Sample(st)
            g = backend.EndCapture()
            for _ in range(steps):
                backend.ReplayGraph(g)
            backend.Synchronize()
            backend.DestroyGraph(g)
        else:
            for _ in range(steps):
                s.Sample(st)
        return [[t.Id for t in row] for row in s.Read(0, steps)]

    direct, replayed = run(False), run(True)
    assert direct == replayed
    assert any(direct[i] != direct[i + 1] for i in range(steps - 1)), "penalties and the step counter must change the draws"


@pytest.mark.gpu
def test_generate_with_sampler(backend, dev, orc):
    """CharGpt.Generate with a TokenSampler in the recorded step (CharGpt.cs:261-308): prefill samples from the last
    of several positions, the graph replays the sampling kernels, a context reset samples again from a prefill."""
    from nn_b200.gpt import GptConfig
    from nn_b200.gpt_f32 import GptF32
    from nn_b200.sampling import TokenSampler
    from oracle import model as om
    from oracle.sampler import TokenSampler as OracleSampler
    cfg = GptConfig(vocab=40, dim=32, heads=2, layers=2, ff_dim=128, context=24)
    w = om.make_weights(cfg, seed=21, std=0.3, sinusoid=True)
    B, n_new = 3, 30
    prompt = orc.token_ids((B, 5), 8, cfg.vocab).astype(np.int64)
    o = OracleSampler(B, cfg.vocab, n_new)
    o.temperature, o.top_k, o.top_p, o.repeat, o.seed = 0.7, 12, 0.95, 1.15, 77
    o.set_history([int(t) for t in prompt[0]])
    ref = om.F32Decoder(cfg, w, B)
    exp, exp_resets = ref.generate(prompt, n_new, sampler=o)
    m = GptF32(dev, cfg, w, B, max_steps=12)
    s = TokenSampler(m.be, B, cfg.vocab, n_new)
    s.Temperature, s.TopK, s.TopP, s.RepeatPenalty, s.Seed = 0.7, 12, 0.95, 1.15, 77
    s.SetHistory([int(t) for t in prompt[0]])
    m.set_sampler(s)
    got, resets, trace = m.generate(prompt, n_new, use_graph=True)
    assert resets == exp_resets >= 1
    # identical up to the first draw that differs (a rounding-level difference at a boundary of the running sum)
    same = 0
    while same < n_new and np.array_equal(got[:, same], exp[:, same]):
        assert orc.close(ref.logit_trace[same], trace[same], 1e-4)
        same += 1
    assert same >= n_new // 2, f"draws diverge at step {same}"
    stats = s.Read(0, n_new)
    assert [[t.Id for t in row] for row in stats] == [list(got[:, i]) for i in range(n_new)]
    assert all(0.0 < t.Probability <= 1.0 and t.Entropy >= 0.0 for row in stats for t in row)
