"""TEST INFRASTRUCTURE (not the product): numpy restatement of the reference's sampling head, models/serve.py:23-29
(Head.of) and :31-47 (heads): a row's k largest by numpy's stable argsort and the log-sum-exp at the row's 1/temperature
in float64.  Pinned by the reference's own test of it (test/test_sim.py:2141-2156 states the same two formulas)."""
import numpy as np


def heads(logits, t=None, k=64):
    x = np.asarray(logits, np.float32)
    ids = np.argsort(-x, -1, kind="stable")[:, :k]
    values = np.take_along_axis(x, ids, -1)
    if t is None:
        return values, ids.astype(np.int32)
    scaled = np.float64(x) * np.asarray(t, np.float64).reshape(-1, 1)
    m = scaled.max(1, keepdims=True)
    return values, ids.astype(np.int32), (m + np.log(np.exp(scaled - m).sum(1, keepdims=True)))
