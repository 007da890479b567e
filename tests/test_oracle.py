"""The CPU oracle against the fixtures generated from the unmodified reference (tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest

from conftest import golden
from oracle import bfp, llama


def test_bf16_rounding_is_nearest_even():
    a = np.array([1.0, 1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8, -(1 + 2.0 ** -8), 1 + 2.0 ** -8 + 2.0 ** -20], np.float32)
    assert bfp.bf16_bits(a).tolist() == [0x3F80, 0x3F80, 0x3F82, 0xBF80, 0x3F81]


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_bfp_matches_reference_vectors(fmt):
    g = golden("bfp.npz")
    for name in ("spread", "edge", "wide", "weights"):
        x = bfp.bf16_floats(g[f"{name}.bits"])
        assert np.array_equal(bfp.bfp(x, fmt), g[f"{name}.{fmt}"]), name


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_fields_properties(fmt):
    x = bfp.bf16_floats(golden("bfp.npz")["edge.bits"])
    top, sign, mag = bfp.fields(x, fmt)
    assert mag.max() <= (127 if fmt == "bfp8" else 7)
    assert not sign[mag == 0].any(), "a zero is stored without a sign"
    y = bfp.bfp(bfp.bf16_floats(golden("bfp.npz")["spread.bits"]), fmt)  # (normal numbers: a run of bf16 denormals halves, models/gpt2.py:26)
    assert np.array_equal(bfp.bfp(y, fmt), y), "quantising twice changes nothing"


def test_topk_matches_reference_vectors():
    g = golden("topk.npz")
    for i in range(len(g.files) // 3):
        x = bfp.bf16_floats(g[f"{i}.bits"])
        vals, ids = llama.topk(x, int(g[f"{i}.k"]))
        assert np.array_equal(ids, g[f"{i}.ids"])


def test_touched_known_answer():
    # the reference's own expectation (test/test_sim.py:1528-1529): expert 5, weighted 0, is not listed
    ids = np.array([[0, 3], [5, 3], [7, 1]])
    w = np.array([[0.5, 0.5], [0, 0], [0.25, 0.75]], np.float32)
    experts, weights = llama.touched(ids, w, 8)
    assert experts[:, 0].tolist() == [0, 1, 3, 7, 8, 8]
    assert weights[2, :, 0].tolist() == [0.5, 0, 0] and weights[3, :, 0].tolist() == [0, 0, 0.25]


def test_moe_matches_reference_vectors():
    g = golden("moe.npz")
    w = {k: bfp.bf16_floats(g[k]) for k in ("router", "experts.gate_up", "experts.down")}
    c = llama.model(dim=64, k=4)
    for n in (1, 3, 8, 40, 160):
        h, live = bfp.bf16_floats(g[f"h{n}"]), np.float32(np.arange(n) != 1).reshape(n, 1)
        assert np.allclose(llama.moe(h, w, c, live=live), g[f"y{n}"], rtol=1e-12, atol=1e-12)


def _checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(k.encode())
        h.update(np.ascontiguousarray(w[k], np.float32).tobytes())
    return h.hexdigest()


MODELS = {
    "dense_bfp8": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, ffn=512, places=64), "bfp8", None),
    "dense_bfp4": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, ffn=512, places=64), "bfp4", None),
    "smol_shape": (dict(dim=576, heads=9, kv=3, layers=2, eps=1e-5, theta=10000.0, vocab=1024, ffn=1536, places=64), "bfp8", None),
    "slots4": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=500000.0, vocab=512, ffn=512, places=64), "bfp8", 4),
    "moe_top2": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, experts=8, k=2, moe=128, places=64), "experts", None),
    "qwen_moe": (dict(dim=256, heads=4, kv=2, head_dim=128, layers=2, eps=1e-6, theta=1000000.0, vocab=512, experts=16, k=4, moe=64,
                      places=64, qk_norm=True), "bfp8", 4),
}


def golden_model(name):
    """(config, raw bf16 weights, quantised float32 weights) of a golden model case, regenerated from its seed."""
    fields, mode, slots = MODELS[name]
    c = llama.model(**fields)
    raw = llama.synthetic(c, seed=11, norm_sigma=0.1, embed_sigma=1.0)
    assert _checksum(raw) == str(golden("models.npz")[f"{name}.checksum"]), "seeded weights differ from the ones the fixture was made with"
    return c, raw, llama.arrays(raw, llama.precision(c, mode)), slots


@pytest.mark.parametrize("name", [n for n, v in MODELS.items() if v[2] is None])
def test_forward_matches_reference_vectors(name):
    g = golden("models.npz")
    c, _, w, _ = golden_model(name)
    ids, want, kv = g[f"{name}.ids"].tolist(), g[f"{name}.logits"], llama.kv_cache(c, 32)
    for i in range(5):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        got = llama.forward(new, places, w, c, kv)
        assert np.allclose(got[0], want[i], rtol=1e-9, atol=1e-9), (name, i)


@pytest.mark.parametrize("name", [n for n, v in MODELS.items() if v[2]])
def test_batched_decode_matches_reference_vectors(name):
    g = golden("models.npz")
    c, _, w, slots = golden_model(name)
    size, kv = 32, llama.kv_cache(c, 32 * slots)
    for u, p in enumerate(g[f"{name}.prompts"]):
        p = [int(t) for t in p if t >= 0]
        part = [layer[:, u * size:(u + 1) * size] for layer in kv]
        assert np.allclose(llama.forward(p, range(len(p)), w, c, part)[0], g[f"{name}.prefill"][u], rtol=1e-9, atol=1e-9)
    for i in range(4):
        got = llama.forward(g[f"{name}.step{i}.ids"].tolist(), g[f"{name}.step{i}.places"].tolist(), w, c, kv, slots)
        assert np.allclose(got, g[f"{name}.steps"][i], rtol=1e-9, atol=1e-9), (name, i)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_c_restatement_equals_the_numpy_one(fmt):
    from oracle import build
    g = golden("bfp.npz")
    for name in ("spread", "edge", "wide", "weights"):
        x = bfp.bf16_floats(g[f"{name}.bits"])
        assert np.array_equal(build.bfp_values(x, fmt).astype(np.float64), g[f"{name}.{fmt}"]), name
    big = np.random.default_rng(1).normal(0, 0.02, (512, 1024)).astype(np.float32)
    assert np.array_equal(build.bfp_values(big, fmt), bfp.bfp(big, fmt).astype(np.float32))


def test_sampling_head_restated():
    """oracle.serve.heads against the formulas the reference's own test states (test/test_sim.py:2152-2155)."""
    from oracle import serve as oserve
    rng = np.random.default_rng(3)
    x, ts = rng.normal(0, 3, (3, 512)).astype(np.float32), [1.0, 1 / 0.7, 2.0]
    x[1, 5] = x[1, 505] = x[1].max() + 1
    values, ids, lse = oserve.heads(x, ts)
    want = np.argsort(-x, -1, kind="stable")[:, :64]
    scaled = np.float64(x) * np.array(ts)[:, None]
    exact = scaled.max(1) + np.log(np.exp(scaled - scaled.max(1, keepdims=True)).sum(1))
    assert np.array_equal(ids, want) and np.array_equal(values, np.take_along_axis(x, want, -1)) and ids[1, 0] == 5 and ids[1, 1] == 505
    assert np.allclose(lse[:, 0], exact, rtol=1e-12)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_block_float_kv_cache_matches_reference_vectors(fmt):
    """The restatement with a block-float KV cache (models/llama.py:127-128) against the reference's logits."""
    import copy
    g = golden("kv.npz")
    c, _, w, _ = golden_model("dense_bfp8")
    c = copy.copy(c)
    c.cache = fmt
    ids, want, kv = g[f"{fmt}.ids"].tolist(), g[f"{fmt}.logits"], llama.kv_cache(c, 32)
    for i in range(5):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        got = llama.forward(new, places, w, c, kv)
        assert np.allclose(got[0], want[i], rtol=1e-9, atol=1e-9), (fmt, i)


def test_chunked_prefill_matches_reference_vectors():
    g = golden("prefill.npz")
    c, _, w, _ = golden_model("dense_bfp8")
    for tokens in (1, 4, 13):
        got = llama.prefill(g["ids"].tolist(), w, c, llama.kv_cache(c, 32), tokens)
        assert np.allclose(got[0], g[f"logits{tokens}"], rtol=1e-9, atol=1e-9), tokens


def test_experts_by_expert_is_experts():
    # the grouped evaluation the large-shape GPU tests use gives what the reference's per-token loop gives
    g = golden("moe.npz")
    w = {k: bfp.bf16_floats(g[k]) for k in ("router", "experts.gate_up", "experts.down")}
    c = llama.model(dim=64, k=4)
    h = bfp.bf16_floats(g["h40"]).astype(np.float64)
    want = llama.moe(h, w, c)
    c.by_expert = True
    assert np.allclose(llama.moe(h, w, c), want, rtol=1e-10, atol=1e-12)


def test_group_known_answer():
    # three rows choosing two of four values: value 0 once, 1 twice, 3 three times; runs of whole tiles of 32 in value order
    order, tiles, places = llama.group(np.array([[3, 1], [0, 3], [1, 3]]), 4)
    t, rp = -(-6 // 32) + 4, 32
    assert len(order) == 32 * t and len(tiles) == t and len(places) == 2 * rp
    assert tiles.tolist() == [0, 1, 3, 4, 4], "value 2 is picked by nobody and takes no tile; 4 marks the tiles past those used"
    assert order[0] == 1 and order[32:34].tolist() == [0, 2] and order[64:67].tolist() == [0, 1, 2]
    assert places[:3].tolist() == [64, 0, 33] and places[rp:rp + 3].tolist() == [32, 65, 66]
