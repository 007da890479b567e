"""The general operator surface (Tensor.of, + - * /, relu, softmax, reductions, @, views, gather / put, topk, touched,
attend) against numpy, in the shape of the reference's own operator tests (test/test_sim.py:523-680, 1471-1529, 2063-2079)."""
import numpy as np
import pytest

from conftest import golden
from oracle import bfp, llama as ollama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt(cuda):
    from ferrite_b200.tensor import Runtime
    return Runtime(0)


def bf16(a):
    return bfp.bf16_round(np.asarray(a, np.float32)).astype(np.float64)


def value(t):
    return t.numpy().astype(np.float64)


def close(t, want, tol=2 ** -7):
    got = value(t).reshape(np.shape(want))
    assert np.allclose(got, want, rtol=tol, atol=tol), f"off by up to {np.abs(got - want).max()}"


def test_of_rounds_to_nearest_even_and_round_trips(rt):
    from ferrite_b200.tensor import Tensor
    data = [[1.0, 1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8], [-2.5, 0.0, 3e38]]
    t = Tensor.of(rt, data)
    assert t.shape == (1, 2, 3) and np.array_equal(value(t)[0], bf16(data))
    assert Tensor.frombytes(rt, 2, 3, t.tobytes()).tolist() == t.tolist()
    i = Tensor.of(rt, [[1, -7, 2 ** 20]], "int32")
    assert i.tolist() == [[1, -7, 2 ** 20]]
    with pytest.raises(AssertionError):
        Tensor.frombytes(rt, 1, 16, bytes(16), dtype="bfp8")  # a block float is made on the device, by cast


def test_elementwise_broadcast_and_fusion(rt):
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(2)
    a, b, row, col = bf16(rng.normal(0, 1, (2, 40, 48))), bf16(rng.normal(0, 1, (2, 40, 48))), bf16(rng.normal(0, 1, (1, 48))), bf16(rng.normal(0, 1, (40, 1)))
    ta, tb, tr, tc = (Tensor.of(rt, x.tolist()) for x in (a, b, row, col))
    before = rt.launches
    y = ((ta + tb * tr - tc) * 0.5).relu().realize()
    assert rt.launches == before + 1, "one expression, one kernel"
    close(y, np.maximum((a + b * row - col) * 0.5, 0))
    close((ta * 2).exp().log(), a * 2, 2 ** -6)
    close(ta.maximum(tb) - ta.minimum(tb), np.abs(a - b))
    close((ta > tb).where(ta, tb), np.maximum(a, b))
    close(ta.sigmoid(), 1 / (1 + np.exp(-a)))
    close(ta.silu(), a / (1 + np.exp(-a)))
    close(1 / (ta * ta + 1), 1 / (a * a + 1))
    assert (ta.float() + 1).dtype == "fp32" and ((ta < 0) + 0).tolist() == (a < 0).astype(float).tolist()


def test_reductions_softmax_layernorm(rt):
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(3)
    a = bf16(rng.normal(0, 2, (3, 33, 70)))
    t = Tensor.of(rt, a.tolist())
    for axis in (0, 1, 2):
        close(t.float().sum(axis), a.sum(axis, keepdims=True), 1e-4)
        assert np.array_equal(value(t.max(axis)), a.max(axis, keepdims=True))
    close(t.float().mean(), a.mean(keepdims=True), 1e-4)
    e = np.exp(a - a.max(-1, keepdims=True))
    close(t.softmax(), e / e.sum(-1, keepdims=True))
    close(t.float().layernorm(), (a - a.mean(-1, keepdims=True)) / np.sqrt(a.var(-1, keepdims=True) + 1e-5), 1e-3)


def test_matmul_views_and_movement(rt):
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(4)
    a, b = bf16(rng.uniform(-1, 1, (2, 37, 96))), bf16(rng.uniform(-1, 1, (2, 96, 50)))
    ta, tb = Tensor.of(rt, a.tolist()), Tensor.of(rt, b.tolist())
    close((ta @ tb).float() if False else ta.matmul(tb, "fp32"), a @ b, 1e-4)
    close(ta.matmul(Tensor.of(rt, b.transpose(0, 2, 1).tolist()).T, "fp32"), a @ b, 1e-4)  # B read transposed
    close(ta[0].matmul(tb, "fp32"), a[:1] @ b, 1e-4)  # a batch of 1 repeats
    assert np.array_equal(value(ta[:, 5:20, 32:64]), a[:, 5:20, 32:64]) and np.array_equal(value(ta[1]), a[1:2])
    assert np.array_equal(value(ta.reshape(2, 96, 37)), a.reshape(2, 96, 37))
    assert np.array_equal(value(ta.permute(1, 0, 2)), a.transpose(1, 0, 2))
    m = Tensor.of(rt, a[0].tolist())
    assert np.array_equal(value(m.split(3)), a[0].reshape(37, 3, 32).transpose(1, 0, 2))
    assert np.array_equal(value(m.split(3).merge()), a[:1])
    assert np.array_equal(value(m.pad(((1, 2), (0, 3)))), np.pad(a[:1], ((0, 0), (1, 2), (0, 3))))
    assert np.array_equal(value(ta.cat(ta, axis=1)), np.concatenate([a, a], 1))
    assert np.array_equal(value(m.repeat_interleave(3)), np.repeat(a[:1], 3, 0))
    assert np.array_equal(value(m.expand(4, 37, 96)), np.broadcast_to(a[:1], (4, 37, 96)))


def test_block_float_matmul_is_the_matmul_by_its_values(rt):
    # test/test_sim.py:373-388: a cast is numpy's model bit for bit, and x @ w is the matmul by the values w holds
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(5)
    a = bf16(rng.normal(0, 1, (64, 96)) * np.exp(rng.normal(0, 2, (64, 96))))
    for fmt in ("bfp8", "bfp4"):
        assert np.array_equal(value(Tensor.of(rt, a.tolist()).cast(fmt))[0], bfp.bfp(a, fmt))
        for m, k, n in ((1, 768, 2304), (100, 256, 208), (32, 2048, 64)):
            x, w = bf16(rng.normal(0, 1, (m, k))), bf16(rng.normal(0, 1, (k, n)))
            tx, tw = Tensor.of(rt, x.tolist()), Tensor.of(rt, w.tolist()).cast(fmt).realize()
            close(tx.matmul(tw, "fp32"), x @ bfp.bfp(w, fmt), 1e-4)
            same = Tensor.of(rt, bfp.bfp(w, fmt).tolist())
            assert np.array_equal(value(tx @ tw), value(tx.matmul(same.cast(fmt).realize()))), "the values decide, not how they were made"


def test_gather_put(rt):
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(23)
    table = bf16(rng.normal(0, 1, (50, 64)))
    assert np.array_equal(value(Tensor.of(rt, table.tolist()).gather([3, 49, 3, 0]))[0], table[[3, 49, 3, 0]])
    for dtype in ("bf16", "fp32"):  # test/test_sim.py:2067-2076
        cache, x = rng.normal(0, 1, (3, 200, 96)).astype(np.float32), rng.normal(0, 1, (3, 70, 96)).astype(np.float32)
        if dtype == "bf16":
            cache, x = bf16(cache), bf16(x)
        places = [int(p) for p in rng.permutation(200)[:70]]
        places[40] = places[7]
        t = Tensor.of(rt, cache.tolist(), dtype)
        t.put(Tensor.of(rt, [places], "int32"), Tensor.of(rt, x.tolist(), dtype))
        for i, p in enumerate(places):
            cache[:, p] = x[:, i]
        assert np.array_equal(value(t), cache), dtype


def test_topk_and_touched(rt):
    from ferrite_b200.tensor import Tensor
    g = golden("topk.npz")
    for i in range(len(g.files) // 3):
        x = bfp.bf16_floats(g[f"{i}.bits"])
        values, ids = Tensor.of(rt, x.tolist()).topk(int(g[f"{i}.k"]))
        assert np.array_equal(ids.numpy().reshape(g[f"{i}.ids"].shape), g[f"{i}.ids"]), i
        assert np.array_equal(value(values).reshape(g[f"{i}.ids"].shape), np.take_along_axis(x, g[f"{i}.ids"].astype(np.int64), -1)), i
    rng = np.random.default_rng(37)
    x = rng.normal(0, 3, (5, 2560)).astype(np.float32)  # fp32 rows in parts, then their best by labels (test_sim.py:1494-1503)
    x[0, 100] = x[0, 1283] = x[0].max() + 1
    t = Tensor.frombytes(rt, 5, 2560, x.tobytes(), dtype="fp32")
    values, ids = t.topk(64, 4)
    want = np.concatenate([np.argsort(-x[:, p * 640:(p + 1) * 640], -1, kind="stable")[:, :64] + p * 640 for p in range(4)], 1)
    assert np.array_equal(ids.numpy()[0], want)
    values, ids = values.topk(64, labels=ids)
    assert np.array_equal(ids.numpy()[0], np.argsort(-x, -1, kind="stable")[:, :64])
    ids, w = Tensor.of(rt, [[0, 3], [5, 3], [7, 1]], "int32"), Tensor.of(rt, [[0.5, 0.5], [0, 0], [0.25, 0.75]])
    experts, weights = ids.touched(8, w)
    assert experts.numpy()[0, :, 0].tolist() == [0, 1, 3, 7, 8, 8], "expert 5, weighted 0, not listed (test_sim.py:1528-1529)"
    oe, ow = ollama.touched(np.array(ids.tolist()), np.array(w.tolist(), np.float32), 8)
    assert np.array_equal(weights.numpy(), ow)


def test_group(rt):
    # Tensor.group against the restated counting sort, slot for slot: the reference's own case (40 rows, top-4 of 16,
    # test/test_sim.py:1506), one value taking every choice, values nobody picks, a prompt-sized case
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(47)
    x = bf16(rng.normal(0, 1, (40, 16)))
    cases = [(Tensor.of(rt, x.tolist()).topk(4)[1].numpy()[0], 16), (np.zeros((5, 2), np.int64), 4), (rng.integers(3, 5, (70, 1)), 8),
             (rng.integers(0, 128, (2048, 8)), 128), (np.array([[1]]), 2)]
    for ids, n in cases:
        order, tiles, places = Tensor.of(rt, ids.tolist(), "int32").group(n)
        want = ollama.group(ids, n)
        assert order.shape == (1, 1, len(want[0])) and tiles.shape == (1, len(want[1]), 1) and places.shape == (1, 1, len(want[2]))
        for got, w in zip((order, tiles, places), want):
            assert np.array_equal(got.numpy().reshape(-1), w), (ids.shape, n)
        # what it is for: each expert's rows are whole tiles, and places lead every choice back to its row
        rows, k = ids.shape
        rp, o, pl, tl = -(-rows // 32) * 32, want[0], want[2], want[1]
        for r in range(rows):
            for j in range(k):
                s = pl[j * rp + r]
                assert o[s] == r and tl[s // 32] == ids[r, j]


def test_attend(rt):
    # the shape of the reference's test_attend (test/test_sim.py:641-680): several rows of queries each with its place,
    # a key head serving two query heads (a repeat read in place), one column of places for all, a sliding window
    from ferrite_b200.tensor import Tensor
    rng = np.random.default_rng(43)
    for e, rows, hd, keys, rep, shared, window, lo, hi in ((2, 40, 64, 64, 1, False, 0, 0, 64), (4, 8, 64, 96, 2, False, 0, 0, 96),
                                                           (2, 33, 128, 128, 1, True, 0, 0, 128), (3, 70, 64, 40, 1, True, 0, 0, 40),
                                                           (2, 40, 128, 200, 1, False, 50, 60, 200), (2, 8, 64, 256, 1, False, 0, 200, 256),
                                                           (4, 8, 64, 1024, 2, False, 0, 0, 1024)):
        q, k, v = (bf16(rng.normal(0, 1, s)) for s in ((e, rows, hd), (e // rep, keys, hd), (e // rep, keys, hd)))
        places = rng.integers(lo, hi, (1 if shared else e, rows, 1))
        mask = np.where((np.arange(keys) > places) | ((np.arange(keys) <= places - window) if window else False), -1e9, 0)
        tq, tk, tv = (Tensor.of(rt, x.tolist()) for x in (q, k, v))
        if rep > 1:
            tk, tv = tk.repeat_interleave(rep), tv.repeat_interleave(rep)
        out = tq.attend(tk, tv, Tensor.of(rt, places.tolist(), "int32"), window)
        s = q @ np.repeat(k, rep, 0).transpose(0, 2, 1) + mask
        p = np.exp(s - s.max(-1, keepdims=True))
        close(out, p / p.sum(-1, keepdims=True) @ np.repeat(v, rep, 0), 0.01)
