"""TEST INFRASTRUCTURE ONLY.  Host restatement of the reference's TokenSampler (src/NeuralSharp/Sampling.cs:16-183)
over the C oracle's SampleRows / PenalizeRows / HistoryPush, for the parity tests of the on-device sampler."""
from __future__ import annotations

import numpy as np

from . import oracle as O


class TokenSampler:
    def __init__(self, rows: int, vocabulary: int, max_steps: int, history_capacity: int = 256):
        self.rows, self.vocabulary, self.max_steps, self.capacity = rows, vocabulary, max_steps, history_capacity
        self.ids = np.zeros(rows, np.float32)
        self.stats = np.zeros(max_steps * rows * 13, np.float32)
        self.step = 0
        self.history = np.zeros((rows, history_capacity), np.float32)
        self.length = 0
        self.temperature, self.top_k, self.top_p, self.min_p = 1.0, 0, 1.0, 0.0
        self.repeat, self.last_n, self.presence, self.frequency, self.seed = 1.0, 64, 0.0, 0.0, 0

    def set_history(self, tokens) -> None:
        self.history[:] = 0
        for t in range(max(0, len(tokens) - self.capacity), len(tokens)):
            self.history[:, t % self.capacity] = tokens[t]
        self.length = len(tokens)

    def sample(self, logits, steps: int = 1) -> np.ndarray:
        v = self.vocabulary
        src = np.ascontiguousarray(logits, np.float32).reshape(-1)
        stride, offset = steps * v, (steps - 1) * v
        last_n = min(self.last_n, self.capacity)
        if last_n > 0 and (self.repeat != 1.0 or self.presence != 0.0 or self.frequency != 0.0):
            src = O.penalize_rows(src, self.history, self.length, self.rows, v, stride, offset, self.capacity, last_n, self.repeat,
                                  self.presence, self.frequency).reshape(-1)
            stride, offset = v, 0
        self.ids, _ = O.sample_rows(src, self.step, self.rows, v, stride, offset, self.temperature, self.top_k, self.top_p, self.min_p,
                                    self.seed, stats=self.stats)
        O.history_push(self.ids, self.history, self.length, self.capacity)
        self.length += 1
        self.step += 1
        return self.ids.astype(np.int64)

    def read(self, from_step: int, to_step: int) -> np.ndarray:
        """[steps, rows, 13] statistics."""
        n = self.rows * 13
        return self.stats[from_step * n:to_step * n].reshape(to_step - from_step, self.rows, 13)
