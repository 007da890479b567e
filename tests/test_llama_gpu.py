"""The decoder through the public surface (ferrite_b200.llama.forward on Tensors, replayed by jit) against the golden
logits the unmodified reference produced (tests/golden/make_golden.py), the way the reference's own test_kv_cache and
test_batched_decode check it (test/test_sim.py:1451-1469, 2109-2132): teacher-forced with the reference's picks."""
import numpy as np
import pytest

from conftest import golden
from test_oracle import MODELS, golden_model

pytestmark = pytest.mark.gpu

# logits within 2% of the reference logits' span and the same greedy token (the reference's bound for its 8B-shape
# check, test/test_sim.py:1949); the picks are compared only where the reference's top two are further apart than that
TOL = 0.02


def agrees(got, want):
    span = np.ptp(want)
    err = np.abs(got - want).max()
    top2 = np.sort(want)[-2:]
    return err <= TOL * span and (got.argmax() == want.argmax() or top2[1] - top2[0] <= 2 * err), (err / span, int(got.argmax()), int(want.argmax()))


@pytest.fixture(scope="module")
def rt(cuda):
    from ferrite_b200.tensor import Runtime
    return Runtime(0)


@pytest.mark.parametrize("name", ["dense_bfp8", "dense_bfp4", "smol_shape"])
def test_decode_with_kv_cache_and_replay(rt, name):
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor, jit
    g = golden("models.npz")
    c, raw, _, _ = golden_model(name)
    prec = llama.precision(c, MODELS[name][1])
    t = llama.upload(rt, raw, prec)
    assert t["layers.0.qkv_proj"].dtype == "bfp8" and t["layers.0.gate_up_proj"].dtype == ("bfp4" if name == "dense_bfp4" else "bfp8")
    kv = llama.kv_cache(c, 32, llama.zeros(rt))
    on = lambda row: Tensor.of(rt, [row], "int32")
    step = jit(lambda ids, places: llama.forward(ids, places, t, c, kv))
    ids, want = g[f"{name}.ids"].tolist(), g[f"{name}.logits"]
    for i in range(5):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        out = llama.forward(on(new), on(places), t, c, kv) if i == 0 else step(on(new), on(places))
        ok, detail = agrees(llama.logits(out), want[i])
        assert ok, (name, i, detail)


def test_batched_decode_with_slots(rt):
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor, jit
    name = "slots4"
    g = golden("models.npz")
    c, raw, _, slots = golden_model(name)
    t = llama.upload(rt, raw, llama.precision(c, MODELS[name][1]))
    size = 32
    kv = llama.kv_cache(c, size * slots, llama.zeros(rt))
    on = lambda row: Tensor.of(rt, [row], "int32")
    for u, p in enumerate(g[f"{name}.prompts"]):  # each prompt into its own rows of the shared caches
        p = [int(v) for v in p if v >= 0]
        part = [layer[:, u * size:(u + 1) * size, :] for layer in kv]
        out = llama.forward(on(p), on(list(range(len(p)))), t, c, part)
        ok, detail = agrees(llama.logits(out), g[f"{name}.prefill"][u])
        assert ok, (u, detail)
    step = jit(lambda ids, places: llama.forward(ids, places, t, c, kv, slots))
    for i in range(4):
        got = step(on(g[f"{name}.step{i}.ids"].tolist()), on(g[f"{name}.step{i}.places"].tolist())).numpy()[0]
        for u in range(slots):
            if i == 2 and u == 1:
                continue  # a free slot's token: its logits are not anyone's
            ok, detail = agrees(got[u], g[f"{name}.steps"][i][u])
            assert ok, (i, u, detail)


def test_replayed_step_is_the_step(rt):
    # a replayed step computes bit for bit what the step computes op by op (the reference's claim for jit, test_sim.py:1552)
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor, jit
    c, raw, _, _ = golden_model("dense_bfp8")
    t = llama.upload(rt, raw, llama.precision(c, "bfp8"))
    on = lambda row: Tensor.of(rt, [row], "int32")
    outs = []
    for replay in (False, True):
        kv = llama.kv_cache(c, 32, llama.zeros(rt))
        step = jit(lambda ids, places: llama.forward(ids, places, t, c, kv))
        run = step if replay else (lambda ids, places: llama.forward(ids, places, t, c, kv).realize())
        outs.append([run(on([7 + i]), on([i])).numpy().copy() for i in range(5)])
    assert all(np.array_equal(a, b) for a, b in zip(*outs))


def test_matmul_indexed(rt):
    # x.matmul(w, index=ids): batch entry b is x by the matrix ids picks, one that picks none (16) zeros; each entry equal
    # to the plain matmul by its expert (the reference's test_matmul_indexed, test/test_sim.py:414-429), in bfp8 and bfp4
    from ferrite_b200.tensor import Tensor
    from oracle import bfp
    rng = np.random.default_rng(29)
    experts = bfp.bf16_round(rng.normal(0, 0.1, (16, 128, 256)).astype(np.float32))
    for fmt in ("bfp8", "bfp4"):
        w = Tensor.of(rt, experts.tolist()).cast(fmt).realize()
        for n in (1, 8, 40):
            x = bfp.bf16_round(rng.normal(0, 1, (n, 128)).astype(np.float32))
            ids = rng.integers(0, 16, (6, 1))
            ids[-1, 0] = 16
            got = Tensor.of(rt, x.tolist()).matmul(w, "fp32", index=Tensor.of(rt, ids.tolist(), "int32")).numpy()
            for b, e in enumerate(ids[:, 0]):
                want = x.astype(np.float64) @ bfp.bfp(experts[e], fmt) if e < 16 else np.zeros((n, 256))
                assert np.abs(got[b] - want).max() <= 2e-5 * max(np.abs(want).max(), 1), (fmt, n, b)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_moe_block(rt, fmt):
    # llama.moe on its own against the numpy restatement (the reference's test_moe, test/test_sim.py:1520-1527): router
    # top-k on the device, touched experts, SwiGLUs weighted and summed; a free slot's row (live 0) gives zeros
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    from oracle import bfp, llama as ollama
    rng = np.random.default_rng(31)
    bf = lambda a: bfp.bf16_round(np.asarray(a, np.float32))
    w = {"router": bf(rng.normal(0, 0.5, (64, 16))), "experts.gate_up": bf(rng.normal(0, 0.1, (16, 64, 256))), "experts.down": bf(rng.normal(0, 0.1, (16, 128, 64)))}
    wq = dict(w) | {k: bfp.bfp_f32(w[k], fmt) for k in ("experts.gate_up", "experts.down")}
    t = {k: Tensor.of(rt, v.tolist()) for k, v in w.items()}
    t |= {k: t[k].cast(fmt).realize() for k in ("experts.gate_up", "experts.down")}
    c, oc = llama.model(dim=64, k=4), ollama.model(dim=64, k=4)
    for n in (1, 3, 8, 40, 160):  # (160: the grouped form, each expert's tokens in whole tiles, Tensor.group)
        h, live = bf(rng.normal(0, 1, (n, 64))), np.float32(np.arange(n) != 1).reshape(n, 1)
        got = llama.moe(Tensor.of(rt, h.tolist()), t, c, live=Tensor.of(rt, live.tolist())).realize().numpy()[0]
        want = ollama.moe(h, wq, oc, live=live)
        assert np.abs(got - want).max() < 0.02 * np.abs(want).max() and not got[1:2].any(), (n, np.abs(got - want).max(), np.abs(want).max())


def test_mixture_decoders(rt):
    # two-block mixtures decoding from a replay: Mixtral-like (top-2 of 8, experts in bfp4) and Qwen3-like (QK-norm, top-4
    # of 16, bfp8, four slots), against the reference's golden logits
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor, jit
    g = golden("models.npz")
    on = lambda row: Tensor.of(rt, [row], "int32")
    name = "moe_top2"
    c, raw, _, _ = golden_model(name)
    t = llama.upload(rt, raw, llama.precision(c, MODELS[name][1]))
    assert t["layers.0.experts.gate_up"].dtype == "bfp4" and t["layers.0.qkv_proj"].dtype == "bfp8"
    kv = llama.kv_cache(c, 32, llama.zeros(rt))
    step = jit(lambda ids, places: llama.forward(ids, places, t, c, kv))
    ids, want = g[f"{name}.ids"].tolist(), g[f"{name}.logits"]
    for i in range(5):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        out = llama.forward(on(new), on(places), t, c, kv) if i == 0 else step(on(new), on(places))
        ok, detail = agrees(llama.logits(out), want[i])
        assert ok, (name, i, detail)
    name = "qwen_moe"
    c, raw, _, slots = golden_model(name)
    t = llama.upload(rt, raw, llama.precision(c, MODELS[name][1]))
    size = 32
    kv = llama.kv_cache(c, size * slots, llama.zeros(rt))
    for u, p in enumerate(g[f"{name}.prompts"]):
        p = [int(v) for v in p if v >= 0]
        out = llama.forward(on(p), on(list(range(len(p)))), t, c, [layer[:, u * size:(u + 1) * size, :] for layer in kv])
        ok, detail = agrees(llama.logits(out), g[f"{name}.prefill"][u])
        assert ok, (name, "prefill", u, detail)
    step = jit(lambda ids, places: llama.forward(ids, places, t, c, kv, slots))
    for i in range(4):
        got = step(on(g[f"{name}.step{i}.ids"].tolist()), on(g[f"{name}.step{i}.places"].tolist())).numpy()[0]
        for u in range(slots):
            if not (i == 2 and u == 1):
                ok, detail = agrees(got[u], g[f"{name}.steps"][i][u])
                assert ok, (name, i, u, detail)


@pytest.mark.parametrize("tokens", [4, 13])
def test_chunked_prefill(rt, tokens):
    """A 13-token prompt in chunks (models/llama.py:498-504) against the reference's logits for the same chunks."""
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    g = golden("prefill.npz")
    c, raw, _, _ = golden_model("dense_bfp8")
    t = llama.upload(rt, raw, llama.precision(c, "bfp8"))
    kv = llama.kv_cache(c, 32, llama.zeros(rt))
    out = llama.prefill(g["ids"].tolist(), t, c, kv, tokens, lambda row: Tensor.of(rt, [row], "int32"))
    ok, detail = agrees(llama.logits(out), g[f"logits{tokens}"])
    assert ok, detail
