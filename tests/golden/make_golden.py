"""Generate the golden fixtures in this folder from the UNMODIFIED reference (alkinun/ferrite).

Run where a checkout of the reference is at hand:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports the reference's models/gpt2.py and models/llama.py (numpy branch; nothing is compiled),
(1) checks that the restatement under oracle/ reproduces the reference on every case (this is what
"parity pinned" means), and (2) writes the reference's outputs as small .npz files.  The tests then
check the oracle and the CUDA path against these files without needing the reference.

Inputs are seeded; weights of the model cases are regenerated from their seed by
oracle.llama.synthetic and guarded by a checksum stored beside the expected logits.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
assert len(sys.argv) > 1, "usage: make_golden.py <path to the reference checkout>"
REF = sys.argv[1]
sys.path[:0] = [REF, os.path.join(REF, "models"), ROOT]

import gpt2  # noqa: E402  (reference)
import llama  # noqa: E402  (reference)
from oracle import bfp as obfp  # noqa: E402
from oracle import llama as ollama  # noqa: E402


def checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(k.encode())
        h.update(np.ascontiguousarray(w[k], np.float32).tobytes())
    return h.hexdigest()


def bfp_cases():
    """Inputs for the pack/unpack parity: the reference test's own distribution (test/test_sim.py:381,
    seed 5, exponents spread wide inside each run) plus rows built to hit every branch of the rounding."""
    rng = np.random.default_rng(5)
    spread = rng.normal(0, 1, (64, 96)) * np.exp(rng.normal(0, 2, (64, 96)))
    rows = [np.zeros(16), -np.zeros(16)]
    rows.append(np.r_[1.0, -1.0, 0.0, -0.0, 2.0 ** -9, -(2.0 ** -9), 2.0 ** -8, 2.0 ** -7, 255 / 256, 1.9921875, 1.99, 1.5, 0.75, 0.375, 3e-5, -1e-9])
    rows.append(np.r_[1.9921875, [1.9921875 * 2.0 ** -s for s in range(1, 9)], [-(1 + 2.0 ** -7) * 2.0 ** -s for s in range(7)]])  # largest mantissa: carry clamps
    rows.append(np.array([(1 + j / 128) for j in range(16)]))  # every low mantissa at shift 0
    rows.append(np.array([(1 + (8 * j + 4) / 128) * 2.0 ** -(j % 5) for j in range(16)]))  # ties at several shifts
    rows.append(np.array([1e-39 * (j + 1) for j in range(16)]))  # bf16 denormals only: exponent field 0
    rows.append(np.r_[1e-38, [1e-39 * (j + 1) for j in range(15)]])  # denormals beside the smallest normals
    rows.append(np.array([3e38 / (j + 1) for j in range(16)]))  # near the top of the range
    rows.append(np.array([(-1) ** j * 2.0 ** (j - 8) for j in range(16)]))  # one value per exponent
    for sh in range(10):  # a value exactly `sh` exponents below the run's top, mantissa bits all set and all clear
        rows.append(np.r_[1.0, [1.9921875 * 2.0 ** -sh] * 5, [-(2.0 ** -sh)] * 5, [1.5 * 2.0 ** -sh] * 5])
    edge = np.stack(rows)
    edge = np.concatenate([edge, -edge, edge[:, ::-1]], 0)
    wide = np.random.default_rng(6).normal(0, 1, (32, 256)) * 10.0 ** np.random.default_rng(7).integers(-20, 20, (32, 256))
    weights = np.random.default_rng(8).normal(0, 0.02, (48, 64))
    return {"spread": spread, "edge": edge, "wide": wide, "weights": weights}


def make_bfp():
    out = {}
    for name, a in bfp_cases().items():
        bits = gpt2.bf16_bits(a)
        assert np.array_equal(bits, obfp.bf16_bits(a)), name
        out[f"{name}.bits"] = bits
        for fmt in ("bfp8", "bfp4"):
            want = gpt2.bfp(a, fmt)
            assert np.array_equal(want, obfp.bfp(a, fmt)), (name, fmt)
            assert np.array_equal(want, obfp.bfp(gpt2.bf16_floats(bits), fmt)), (name, fmt)
            out[f"{name}.{fmt}"] = want.astype(np.float64)
    np.savez_compressed(os.path.join(HERE, "bfp.npz"), **out)
    print("bfp.npz", {k: v.shape for k, v in out.items() if k.endswith(".bits")})


def make_topk():
    """The numpy halves of the reference's test_topk (test/test_sim.py:1479-1487): ties, -0 against 0."""
    rng, out = np.random.default_rng(37), {}
    for i, (batch, rows, cols, k) in enumerate(((1, 1, 128, 8), (1, 3, 16, 4), (1, 40, 40, 1), (2, 33, 256, 32), (1, 64, 8, 2), (1, 128, 128, 8))):
        x = rng.normal(0, 2, (batch, rows, cols))
        x[0, -1, :3], x[0, -1, 3:] = [-0.0, 0.0, -0.0], -np.abs(x[0, -1, 3:]) - 1
        x[0, 0, min(9, cols - 1)] = x[0, 0, 3] = x[0, 0].max()
        bits = gpt2.bf16_bits(x)
        x = gpt2.bf16_floats(bits)
        f = llama.fns(x)
        vals, ids = f.topk(x, k)
        ovals, oids = ollama.topk(x, k)
        assert np.array_equal(ids, oids) and np.array_equal(vals, ovals)
        out[f"{i}.bits"], out[f"{i}.ids"], out[f"{i}.k"] = bits, ids.astype(np.int32), np.int32(k)
    np.savez_compressed(os.path.join(HERE, "topk.npz"), **out)
    print("topk.npz", len(out) // 3, "cases")


def ref_weights(c, w):
    """oracle.synthetic's weights in the reference's naming (adds `turn`)."""
    cos, sin, turn = llama.rotary(c, c.places)
    assert np.array_equal(cos, w["cos"]) and np.array_equal(sin, w["sin"]), "rotary tables differ from the reference's"
    return dict(w) | {"turn": turn}


MODELS = {
    # name: (config fields, precision mode, slots)
    "dense_bfp8": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, ffn=512, places=64), "bfp8", None),
    "dense_bfp4": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, ffn=512, places=64), "bfp4", None),
    "smol_shape": (dict(dim=576, heads=9, kv=3, layers=2, eps=1e-5, theta=10000.0, vocab=1024, ffn=1536, places=64), "bfp8", None),
    "slots4": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=500000.0, vocab=512, ffn=512, places=64), "bfp8", 4),
    "moe_top2": (dict(dim=256, heads=4, kv=2, layers=2, eps=1e-5, theta=10000.0, vocab=512, experts=8, k=2, moe=128, places=64), "experts", None),
    "qwen_moe": (dict(dim=256, heads=4, kv=2, head_dim=128, layers=2, eps=1e-6, theta=1000000.0, vocab=512, experts=16, k=4, moe=64,
                      places=64, qk_norm=True), "bfp8", 4),
}


def make_models():
    out = {}
    for name, (fields, mode, slots) in MODELS.items():
        oc = ollama.model(**fields)
        rc = llama.model(**{k: v for k, v in fields.items() if k != "qk_norm"})
        raw = ollama.synthetic(oc, seed=11, norm_sigma=0.1, embed_sigma=1.0)
        prec = ollama.precision(oc, mode)
        # the reference's precision table gives the same formats
        rprec = llama.precision(rc, mode)
        for key, f in prec.items():
            assert rprec[key][0] == f, (key, f, rprec[key])
        ow = ollama.arrays(raw, prec)
        rw = ref_weights(rc, ow)
        for k in raw:  # the reference's own quantiser on the same bf16 weights
            f = llama.weight_format(k, rprec)
            assert f == ollama.weight_format(k, prec), k
            if f != "bf16":
                assert np.array_equal(ow[k], gpt2.bfp(raw[k].reshape(-1, raw[k].shape[-1]), f).reshape(raw[k].shape).astype(np.float32)), k
        rng = np.random.default_rng(3)
        size = 32
        if slots:
            prompts = [[int(t) for t in rng.integers(0, oc.vocab, n)] for n in (3, 2, 5, 1)[:slots]]
            rkv, okv = llama.kv_cache(rc, size * slots, np.zeros), ollama.kv_cache(oc, size * slots)
            seqs, logits = [list(p) for p in prompts], []
            for u, p in enumerate(prompts):  # each prompt into its own rows (test/test_sim.py:2122-2126)
                got = llama.forward(p, range(len(p)), rw, rc, llama.slot(rc, rkv, u, slots))
                part = [kv[:, u * size:(u + 1) * size] for kv in okv]
                mine = ollama.forward(p, range(len(p)), ow, oc, part)
                assert np.allclose(got, mine, rtol=1e-9, atol=1e-9), (name, u)
                logits.append(got[0])
                seqs[u].append(int(got[0].argmax()))
            steps = []
            for i in range(4):
                places = [len(s) - 1 for s in seqs]
                if i == 2: places[1] = size - 1  # a free slot: its token on its part's last row (llama.py:446-447)
                ids = [s[-1] for s in seqs]
                got = llama.forward(ids, places, rw, rc, rkv, slots)
                mine = ollama.forward(ids, places, ow, oc, okv, slots)
                assert np.allclose(got, mine, rtol=1e-9, atol=1e-9), (name, i)
                steps.append(got)
                out[f"{name}.step{i}.ids"], out[f"{name}.step{i}.places"] = np.int32(ids), np.int32(places)
                for u, s in enumerate(seqs):
                    if not (i == 2 and u == 1): s.append(int(got[u].argmax()))
            out[f"{name}.prompts"] = np.array([p + [-1] * (8 - len(p)) for p in prompts], np.int32)
            out[f"{name}.prefill"] = np.stack(logits)
            out[f"{name}.steps"] = np.stack(steps)
        else:
            prompt = [int(t) for t in rng.integers(0, oc.vocab, 5)]
            rkv, okv = llama.kv_cache(rc, size, np.zeros), ollama.kv_cache(oc, size)
            ids, logits = list(prompt), []
            for i in range(5):
                new = ids if i == 0 else ids[-1:]
                places = list(range(len(ids) - len(new), len(ids)))
                got = llama.forward(new, places, rw, rc, rkv)
                mine = ollama.forward(new, places, ow, oc, okv)
                assert np.allclose(got, mine, rtol=1e-9, atol=1e-9), (name, i, np.abs(got - mine).max())
                logits.append(got[0])
                ids.append(int(got[0].argmax()))
            out[f"{name}.ids"] = np.int32(ids)
            out[f"{name}.logits"] = np.stack(logits)
        out[f"{name}.checksum"] = np.array(checksum(raw))
        print(name, "pinned")
    np.savez_compressed(os.path.join(HERE, "models.npz"), **out)


def make_moe():
    """llama.moe alone, numpy branch, with a free slot's row weighted 0 (test/test_sim.py:1520-1527)."""
    rng, out = np.random.default_rng(31), {}
    bf = lambda a: gpt2.bf16_floats(gpt2.bf16_bits(a))
    w = {"router": bf(rng.normal(0, 0.5, (64, 16))), "experts.gate_up": bf(rng.normal(0, 0.1, (16, 64, 128))),
         "experts.down": bf(rng.normal(0, 0.1, (16, 64, 64)))}
    out |= {k: gpt2.bf16_bits(v) for k, v in w.items()}
    rc, oc = llama.model(dim=64, k=4), ollama.model(dim=64, k=4)
    for n in (1, 3, 8, 40, 160):  # (160: more than a decode step's tokens, the grouped form on the device, test_sim.py:1524)
        h, live = bf(rng.normal(0, 1, (n, 64))), np.float32(np.arange(n) != 1).reshape(n, 1)
        want = llama.moe(h, w, rc, live=live)
        assert np.allclose(want, ollama.moe(h, w, oc, live=live), rtol=1e-12, atol=1e-12)
        out[f"h{n}"], out[f"y{n}"] = gpt2.bf16_bits(h), want
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)
    print("moe.npz")


def make_prefill():
    """Chunked prefill (models/llama.py:498-504): the reference's and the restatement's agree chunk size by chunk size,
    and the reference's logits for a 13-token prompt in chunks of 4 are kept."""
    fields, mode, _ = MODELS["dense_bfp8"]
    oc, rc = ollama.model(**fields), llama.model(**fields)
    raw = ollama.synthetic(oc, seed=11, norm_sigma=0.1, embed_sigma=1.0)
    ow = ollama.arrays(raw, ollama.precision(oc, mode))
    rw = ref_weights(rc, ow)
    ids = [int(t) for t in np.random.default_rng(9).integers(0, oc.vocab, 13)]
    out = {"ids": np.int32(ids)}
    for tokens in (1, 4, 13):
        got = llama.prefill(ids, rw, rc, llama.kv_cache(rc, 32, np.zeros), tokens)
        mine = ollama.prefill(ids, ow, oc, ollama.kv_cache(oc, 32), tokens)
        assert np.allclose(got, mine, rtol=1e-9, atol=1e-9), tokens
        out[f"logits{tokens}"] = got[0]
    np.savez_compressed(os.path.join(HERE, "prefill.npz"), **out)
    print("prefill pinned")


def make_kv():
    """A block-float KV cache (models/llama.py:80, 127-128): the reference's numpy branch rounds what it caches with
    gpt2.bfp; the restatement's `cache` option must give the same logits."""
    out = {}
    fields, mode, _ = MODELS["dense_bfp8"]
    for fmt in ("bfp8", "bfp4"):
        oc, rc = ollama.model(**fields), llama.model(**fields)
        oc.cache = fmt
        rc.precision = llama.precision(rc, mode, kv=fmt)
        assert llama.cache_format(rc) == fmt
        raw = ollama.synthetic(oc, seed=11, norm_sigma=0.1, embed_sigma=1.0)
        ow = ollama.arrays(raw, ollama.precision(oc, mode))
        rw = ref_weights(rc, ow)
        rng = np.random.default_rng(5)
        ids, logits = [int(t) for t in rng.integers(0, oc.vocab, 5)], []
        rkv, okv = llama.kv_cache(rc, 32, np.zeros), ollama.kv_cache(oc, 32)
        for i in range(5):
            new = ids if i == 0 else ids[-1:]
            places = list(range(len(ids) - len(new), len(ids)))
            got = llama.forward(new, places, rw, rc, rkv)
            mine = ollama.forward(new, places, ow, oc, okv)
            assert np.allclose(got, mine, rtol=1e-9, atol=1e-9), (fmt, i, np.abs(got - mine).max())
            logits.append(got[0])
            ids.append(int(got[0].argmax()))
        for a, b in zip(rkv, okv):
            assert np.array_equal(a, b), fmt
        out[f"{fmt}.ids"], out[f"{fmt}.logits"] = np.int32(ids), np.stack(logits)
        print("kv cache", fmt, "pinned")
    np.savez_compressed(os.path.join(HERE, "kv.npz"), **out)


if __name__ == "__main__":
    make_bfp()
    make_topk()
    make_moe()
    make_models()
    make_kv()
    make_prefill()
