"""``TokenSampler`` over the C ABI: the Python twin of the reference's class (src/NeuralSharp/Sampling.cs:16-183).

Same constructor arguments, properties, ``SetHistory`` / ``Sample`` / ``Reset`` / ``Read``; same call sequence per
step (PenalizeRows when a penalty is on, SampleRows, HistoryPush, then the length and step counters advance on the
device), so a step that samples can be recorded in a graph exactly as the reference records it.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .backend import NsB200Backend
from .device import Storage

STATS_PER_TOKEN = 13


@dataclass(frozen=True)
class SampledToken:
    """Sampling.cs:8: id, probability, entropy in bits, five (id, probability) alternatives (-1 when fewer exist)."""
    Id: int
    Probability: float
    Entropy: float
    Alternatives: tuple


class TokenSampler:
    def __init__(self, backend: NsB200Backend, rows: int, vocabulary: int, maxSteps: int, historyCapacity: int = 256):
        if historyCapacity <= 0:
            raise ValueError("historyCapacity must be positive")
        self._b = backend
        self.Rows, self.Vocabulary, self.MaxSteps, self.HistoryCapacity = rows, vocabulary, maxSteps, historyCapacity
        self.Ids = backend.Allocate(rows, zeroed=True)
        self._stats = backend.Allocate(maxSteps * rows * STATS_PER_TOKEN, zeroed=True)
        self._step = backend.Allocate(1, zeroed=True)
        self._history = backend.Allocate(rows * historyCapacity, zeroed=True)
        self._historyLength = backend.Allocate(1, zeroed=True)
        self._work = backend.Allocate(rows * vocabulary, zeroed=True)
        self.Temperature = 1.0
        self.TopK = 0
        self.TopP = 1.0
        self.MinP = 0.0
        self.RepeatPenalty = 1.0
        self.RepeatLastN = 64
        self.PresencePenalty = 0.0
        self.FrequencyPenalty = 0.0
        self.Seed = 0

    def SetHistory(self, tokens) -> None:
        """Sampling.cs:71-84: every row gets the same recent tokens, stored modulo the capacity."""
        values = np.zeros((self.Rows, self.HistoryCapacity), np.float32)
        for t in range(max(0, len(tokens) - self.HistoryCapacity), len(tokens)):
            values[:, t % self.HistoryCapacity] = tokens[t]
        self._b.Upload(values.reshape(-1), self._history)
        self._b.Fill(self._historyLength, 1, float(len(tokens)))

    def Sample(self, logits: Storage, steps: int = 1) -> None:
        """Sampling.cs:111-138.  ``logits`` is [rows, vocabulary] or, with ``steps`` > 1, [rows, steps, vocabulary]
        (the last position of each row is sampled); the storage may be larger than that."""
        if logits.count < self.Rows * steps * self.Vocabulary:
            raise ValueError(f"Expected [{self.Rows}, ..., {self.Vocabulary}] logits, got {logits.count} values.")
        b = self._b
        rowStride, rowOffset = steps * self.Vocabulary, (steps - 1) * self.Vocabulary
        lastN = min(self.RepeatLastN, self.HistoryCapacity)
        source = logits
        if lastN > 0 and (self.RepeatPenalty != 1.0 or self.PresencePenalty != 0.0 or self.FrequencyPenalty != 0.0):
            b.PenalizeRows(source, self._work, self._history, self._historyLength, self.Rows, self.Vocabulary, rowStride, rowOffset,
                           self.HistoryCapacity, lastN, self.RepeatPenalty, self.PresencePenalty, self.FrequencyPenalty)
            source, rowStride, rowOffset = self._work, self.Vocabulary, 0
        b.SampleRows(source, self.Ids, self._stats, self._step, self.Rows, self.Vocabulary, rowStride, rowOffset, self.Temperature,
                     self.TopK, self.TopP, self.MinP, self.Seed)
        b.HistoryPush(self.Ids, self._history, self._historyLength, self.Rows, self.HistoryCapacity)
        b.Affine(self._historyLength, self._historyLength, 1, 1.0, 1.0)
        b.Affine(self._step, self._step, 1, 1.0, 1.0)

    def Reset(self) -> None:
        self._b.Fill(self._step, 1, 0.0)
        self._b.Fill(self._historyLength, 1, 0.0)

    def Read(self, fromStep: int, toStep: int):
        """Sampling.cs:148-171: [step][row] tokens of steps [fromStep, toStep), one synchronisation."""
        count = toStep - fromStep
        n = self.Rows * STATS_PER_TOKEN
        raw = self._b.DownloadRange(self._stats, fromStep * n, count * n).reshape(count, self.Rows, STATS_PER_TOKEN)
        return [[SampledToken(int(t[0]), float(t[1]), float(t[2]), tuple((int(t[3 + 2 * a]), float(t[4 + 2 * a])) for a in range(5)))
                 for t in raw[s]] for s in range(count)]

    def Dispose(self) -> None:
        for s in (self.Ids, self._stats, self._step, self._history, self._historyLength, self._work):
            self._b.Return(s)
