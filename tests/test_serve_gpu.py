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


def test_engine_on_the_device_decodes_what_the_oracle_engine_decodes(cuda):
    # five requests through two slots: prompts in chunks (the prefill-shaped attention over a slot's own rows), a shared
    # beginning found in a slot, one recorded step for a token of every slot with only the heads read back - the tokens
    # are those of the same engine driven by the numpy oracle (tests/test_engine.py), greedy
    from ferrite_b200 import llama, serve
    from ferrite_b200.tensor import Runtime
    from test_engine import OracleBackend
    from test_oracle import MODELS, golden_model
    rt, name = Runtime(0), "dense_bfp8"
    c, raw, _, _ = golden_model(name)
    t = llama.upload(rt, raw, llama.precision(c, MODELS[name][1]))
    rng = np.random.default_rng(5)
    system = rng.integers(0, 512, 9).tolist()
    prompts = [system + [3, 4], rng.integers(0, 512, 5).tolist(), system + [8], rng.integers(0, 512, 12).tolist(), system + [3, 4, 5]]
    make = lambda: [serve.Request(p, max_tokens=5 + i) for i, p in enumerate(prompts)]
    want = serve.Engine(OracleBackend(name, 2, 64), slots=2, places=64, chunk=4).run(make())
    engine = serve.Engine(serve.DeviceBackend(rt, t, c, slots=2, places=64), slots=2, places=64, chunk=4)
    got = engine.run(make())
    for i, (g, w) in enumerate(zip(got, want)):
        assert g.made == w.made and g.cached == w.cached, (i, g.made, w.made)
    assert got[2].cached >= len(system)
    # a draw at a temperature from the device's head: the same seed gives the same tokens as from the oracle's head
    sampled = lambda backend: serve.Engine(backend, slots=2, places=64, chunk=8).run([serve.Request(prompts[1], max_tokens=6, temperature=0.7, top_k=8, seed=1)])[0].made
    assert sampled(serve.DeviceBackend(rt, t, c, slots=2, places=64)) == sampled(OracleBackend(name, 2, 64))
