"""Token choice. Order of the filters as in the reference (fusezap/serve/sampling.py:6-10, 61-73): repetition penalty,
temperature, top-k, top-p, softmax in float64, one seeded uniform draw per token.

Greedy rows, temperature rows and rows with top-k or top-p are picked by the device kernels (`Ops.argmax`, `Ops.sample`,
`Ops.sample_filtered`): the host only supplies the request's next uniform number, so the draw is
`searchsorted(cumsum(p), u * sum(p), side="right")` as in sampling.py:73. Rows with a repetition penalty, which needs the
request's history, copy their logits row to the host and go through `host_choice` below, which restates the reference's
filters.
"""
from __future__ import annotations
from typing import Sequence

import numpy as np

from .params import SamplingParams


class RequestSampler:
    """The random stream and history rule of one request."""
    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = np.random.default_rng(params.seed)

    def next_uniform(self) -> float:
        return float(self.rng.random())

    def host_choice(self, logits: np.ndarray, history: Sequence[int]) -> int:
        p = self.params
        lg = repetition_penalty(np.asarray(logits, np.float32), history, p.repetition_penalty)
        if p.greedy:
            return int(np.argmax(lg))
        lg = top_p_filter(top_k_filter(lg.astype(np.float64) / p.temperature, p.top_k), p.top_p)
        prob = softmax(lg)
        u = self.next_uniform()
        return int(np.searchsorted(np.cumsum(prob), u * prob.sum(), side="right").clip(0, len(prob) - 1))


def repetition_penalty(logits: np.ndarray, history: Sequence[int], penalty: float) -> np.ndarray:
    """A seen token's logit is divided by the penalty if positive, multiplied if negative (sampling.py:17-23)."""
    if penalty == 1.0 or len(history) == 0:
        return logits
    out = logits.copy()
    seen = np.unique(np.asarray(history, np.int64))
    v = out[seen]
    out[seen] = np.where(v > 0, v / penalty, v * penalty)
    return out


def top_k_filter(logits: np.ndarray, k: int) -> np.ndarray:
    """Everything below the k-th largest value becomes -inf; ties at that value stay (sampling.py:25-29)."""
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = np.partition(logits, -k)[-k]
    return np.where(logits < kth, -np.inf, logits)


def softmax(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, np.float64)
    e = np.exp(x - np.max(x))
    return e / e.sum()


def top_p_filter(logits: np.ndarray, p: float) -> np.ndarray:
    """Keeps the smallest set of most likely tokens whose mass reaches p, at least one (sampling.py:36-45)."""
    if p >= 1.0:
        return logits
    order = np.argsort(-logits, kind="stable")
    sorted_probs = softmax(logits)[order]
    before = np.cumsum(sorted_probs) - sorted_probs
    drop = np.zeros(logits.shape, bool)
    drop[order] = before >= p
    return np.where(drop, -np.inf, logits)
