"""The sampling head on the device against the numpy restatement (the reference's own test: test/test_sim.py:2141-2156):
the 64 largest of each row and their tokens exactly as numpy's stable argsort has them (ties: the first column), the
log-sum-exp at each row's 1/temperature within fp32's rounding; a small vocabulary (one part) and a large one (parts)."""
import numpy as np
import pytest

from oracle import serve as oserve

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vocab", [512, 49152, 248320])
def test_heads(cuda, vocab):
    from ferrite_b200 import serve
    from ferrite_b200.tensor import Runtime, Tensor
    rt, rng = Runtime(0), np.random.default_rng(3)
    x, ts = rng.normal(0, 3, (3, vocab)).astype(np.float32), [1.0, 1 / 0.7, 2.0]
    x[1, 5] = x[1, vocab - 7] = x[1].max() + 1  # a tie for the first place, far apart
    logits = Tensor.frombytes(rt, 3, vocab, x.tobytes(), dtype="fp32")
    values, ids, lse = serve.heads(logits, Tensor.of(rt, [[t] for t in ts], "fp32"))
    want_values, want_ids, want_lse = oserve.heads(x, ts)
    assert np.array_equal(ids.numpy()[0], want_ids) and np.array_equal(values.numpy()[0], want_values)
    assert np.allclose(lse.numpy()[0], want_lse, rtol=2e-6, atol=0), (lse.numpy()[0].ravel(), want_lse.ravel())
    assert np.array_equal(serve.heads(logits, k=1)[1].numpy()[0][:, 0], want_ids[:, 0])  # each row's best alone
