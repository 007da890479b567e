"""The drop-in boundary, shown: the reference's OWN model code (models/llama.py and models/gpt2.py, unmodified, placed
under oracle/_ref by oracle/make_ref.py) runs its Tensor branch - split, x @ turn for RoPE, put, repeat, attend, topk,
touched, matmul(index=) (models/llama.py:111-146, 277-329, 429-480) - on this library's Tensor, bound by the import the
models make themselves (`from ferrite.tensor import Tensor, jit`, models/llama.py:20), and gives the golden logits the
reference's numpy branch produced (tests/golden/models.npz).  Skipped where oracle/_ref has not been made."""
import numpy as np
import pytest

from conftest import golden
from test_llama_gpu import agrees
from test_oracle import MODELS, golden_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(cuda):
    from oracle import make_ref
    mods = make_ref.modules()
    if mods is None:
        pytest.skip("oracle/_ref is not there: python oracle/make_ref.py, with a checkout of the reference")
    from ferrite_b200.tensor import Runtime
    return (*mods, Runtime(0))


def uploaded(ref, name):
    """The golden model `name` as the reference's own upload puts it on the device: its config object, its precision
    table, its Weight wrappers, its RoPE tables and turn matrix."""
    llama, gpt2, rt = ref
    fields, mode, slots = MODELS[name]
    _, raw, _, _ = golden_model(name)
    c = llama.model(**fields)
    c.precision = llama.precision(c, mode)
    w = {k: v for k, v in raw.items() if k not in ("cos", "sin")}
    w |= dict(zip(("cos", "sin", "turn"), llama.rotary(c, c.places)))
    weights = {k: llama.Weight(lambda v=v: gpt2.bf16_bits(np.asarray(v, np.float32))) for k, v in w.items()}
    return c, llama.upload(rt, weights, c.precision), slots


@pytest.mark.parametrize("name", ["dense_bfp8", "dense_bfp4", "moe_top2"])
def test_reference_forward_decodes_on_this_tensor(ref, name):
    llama, gpt2, rt = ref
    from ferrite_b200.tensor import Tensor
    g = golden("models.npz")
    c, t, _ = uploaded(ref, name)
    assert t["layers.0.qkv_proj"].dtype == "bfp8" and type(t["norm"]) is Tensor
    kv = llama.kv_cache(c, 32, llama.zeros(rt))
    on = lambda row: Tensor.of(rt, [row], "int32")
    step = llama.jit(lambda ids, places: llama.forward(ids, places, t, c, kv))
    ids, want = g[f"{name}.ids"].tolist(), g[f"{name}.logits"]
    for i in range(5):  # a prompt of five, then a token at a time: run, recorded, replayed
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        out = llama.forward(on(new), on(places), t, c, kv) if i == 0 else step(on(new), on(places))
        ok, detail = agrees(llama.logits(out), want[i])
        assert ok, (name, i, detail)


@pytest.mark.parametrize("name", ["slots4", "qwen_moe"])
def test_reference_batched_decode_with_slots(ref, name):
    llama, gpt2, rt = ref
    from ferrite_b200.tensor import Tensor
    g = golden("models.npz")
    c, t, slots = uploaded(ref, name)
    size = 32
    kv = llama.kv_cache(c, size * slots, llama.zeros(rt))
    on = lambda row: Tensor.of(rt, [row], "int32")
    for u, p in enumerate(g[f"{name}.prompts"]):  # each prompt into its own part of the shared caches (the reference's slot())
        p = [int(v) for v in p if v >= 0]
        out = llama.forward(on(p), on(list(range(len(p)))), t, c, llama.slot(c, kv, u, slots))
        ok, detail = agrees(llama.logits(out), g[f"{name}.prefill"][u])
        assert ok, (name, "prefill", u, detail)
    for i in range(4):
        out = llama.forward(on(g[f"{name}.step{i}.ids"].tolist()), on(g[f"{name}.step{i}.places"].tolist()), t, c, kv, slots)
        got = gpt2.values(out)
        for u in range(slots):
            if i == 2 and u == 1:
                continue  # a free slot's token: its logits are not anyone's
            ok, detail = agrees(got[u], g[f"{name}.steps"][i][u])
            assert ok, (name, i, u, detail)
