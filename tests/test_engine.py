"""The slot engine's host logic (admit / fill / advance / take, models/serve.py:247-330) on CPU, its device side played
by the numpy oracle: what several requests sharing slots decode is what each decodes alone, a slot that still holds a
prompt's beginning prefills only the rest, and a finished request's slot is taken by the next one waiting."""
import numpy as np

from oracle import llama as ollama
from oracle import serve as oserve
from test_oracle import golden_model


class OracleBackend:
    def __init__(self, name, slots, places):
        self.c, _, self.w, _ = golden_model(name)
        self.slots, self.part = slots, places
        self.kv = ollama.kv_cache(self.c, slots * places)
        self.prefills = []

    def prefill(self, u, ids, first, t):
        part = [kv[:, u * self.part:(u + 1) * self.part] for kv in self.kv]
        self.prefills.append((u, first, len(ids)))
        out = ollama.forward(ids, list(range(first, first + len(ids))), self.w, self.c, part)
        v, i, l = oserve.heads(out, [t])
        return v[0], i[0], l[0, 0]

    def decode(self, ids, places, ts):
        out = ollama.forward(ids, places, self.w, self.c, self.kv, self.slots)
        v, i, l = oserve.heads(out, ts)
        return [(v[u], i[u], l[u, 0]) for u in range(self.slots)]


def alone(name, ids, n):
    """Greedy decode of one prompt on its own, by the oracle."""
    c, _, w, _ = golden_model(name)
    kv, out, made = ollama.kv_cache(c, 64), None, []
    out = ollama.forward(ids, list(range(len(ids))), w, c, kv)
    for i in range(n):
        made.append(int(out[0].argmax()))
        out = ollama.forward(made[-1:], [len(ids) + i], w, c, kv)
    return made


def test_engine_requests_share_slots_and_prefixes():
    from ferrite_b200.serve import Engine, Request, reach
    assert reach([1, 2, 3], [1, 2, 3]) == 2 and reach([1, 2, 3], [1, 2, 4, 5]) == 2 and reach([], [7]) == 0 and reach([9], [7, 8]) == 0
    rng = np.random.default_rng(5)
    system = rng.integers(0, 512, 9).tolist()
    prompts = [system + [3, 4], rng.integers(0, 512, 5).tolist(), system + [8], rng.integers(0, 512, 12).tolist(), system + [3, 4, 5]]
    backend = OracleBackend("dense_bfp8", slots=2, places=32)
    engine = Engine(backend, slots=2, places=32, chunk=4)
    rs = engine.run([Request(p, max_tokens=5 + i) for i, p in enumerate(prompts)])
    for i, (r, p) in enumerate(zip(rs, prompts)):
        assert r.finish == "length" and r.made == alone("dense_bfp8", p, 5 + i), (i, r.made)
    assert rs[0].cached == 0 and rs[2].cached >= len(system), "the third request found the first one's prompt in its slot"
    assert engine.prefilled == sum(len(p) - r.cached for p, r in zip(prompts, rs)) < sum(map(len, prompts))
    assert all(n <= 4 for _, _, n in backend.prefills), "prompts go in chunk by chunk"
    assert engine.decoded == sum(len(r.made) - 1 for r in rs)


def test_request_sampling_from_the_head():
    from ferrite_b200.serve import Request
    logits = np.array([[2.0, 1.0, 0.0, -1.0] + [-20.0] * 508], np.float32)
    values, ids, lse = oserve.heads(logits, [1 / 0.8])
    assert Request([1], temperature=0).sample(values[0], ids[0], lse[0, 0]) == 0
    r = Request([1], temperature=0.8, seed=3)
    draws = np.bincount([r.sample(values[0], ids[0], lse[0, 0]) for _ in range(4000)], minlength=4)[:4] / 4000
    want = np.exp(logits[0, :4] / 0.8) / np.exp(logits[0] / 0.8).sum()
    assert np.abs(draws - want).max() < 0.03, (draws, want)
    r = Request([1], temperature=0.8, top_k=2, seed=4)
    assert set(r.sample(values[0], ids[0], lse[0, 0]) for _ in range(200)) == {0, 1}
    r = Request([1], max_tokens=3, eos=[7])
    assert not r.take(5, True) and r.take(7, True) and r.finish == "stop" and r.made == [5]
