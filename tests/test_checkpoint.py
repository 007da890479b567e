"""The checkpoint reader on CPU (models/llama.py:376-427, 572-604; models/gpt2.py:34-47): a Hugging Face checkpoint
that the test writes itself (the golden models' weights un-fused and stored out x in under the hub's names, BF16 or
F32, one file or sharded with an index) comes back under the reference's fused names with the same values, and the
oracle fed the loaded weights gives the golden logits."""
import numpy as np
import pytest

from conftest import golden
from oracle import llama as ollama
from test_oracle import MODELS, golden_model


def as_oracle(c, w):
    """{name: Weight} -> float32 arrays as oracle.llama takes them (its wide RoPE tables, v's rows of the q/k norm)."""
    out = {k: v.values() for k, v in w.items() if k not in ("cos", "sin")}
    for k in [k for k in out if k.endswith("qk_norm")]:
        out[k] = np.concatenate([out[k], np.ones((c.kv, 1, out[k].shape[-1]), np.float32)])
        out[k[:-4] + "on"] = np.array([1.0] * (c.heads + c.kv) + [0.0] * c.kv, np.float32).reshape(-1, 1, 1)
    out["cos"], out["sin"] = ollama.rotary(c, c.places)
    return out


@pytest.mark.parametrize("name,dtype,shards", [("dense_bfp8", "BF16", 1), ("dense_bfp8", "F32", 3), ("qwen_moe", "BF16", 2), ("moe_top2", "BF16", 1)])
def test_saved_checkpoint_loads_fused(tmp_path, name, dtype, shards):
    from ferrite_b200 import checkpoint, llama
    fields, mode, slots = MODELS[name]
    c0, raw, _, _ = golden_model(name)
    checkpoint.save(str(tmp_path), llama.model(**fields), raw, dtype, shards)
    c, w = checkpoint.load(str(tmp_path), places=64)
    assert (c.dim, c.heads, c.kv, c.layers, c.vocab, c.experts, c.k, llama.head(c)) == (c0.dim, c0.heads, c0.kv, c0.layers, c0.vocab, c0.experts, c0.k, ollama.head(c0))
    got = as_oracle(c, w)
    for k, v in raw.items():
        assert k in got and np.array_equal(got[k], np.asarray(v, np.float32).reshape(got[k].shape)), k
    cos, sin = llama.rotary(c, c.places)
    assert np.array_equal(w["cos"].values(), cos) and np.array_equal(w["sin"].values(), sin)
    if slots is None:  # the loaded model decodes the golden logits
        g = golden("models.npz")
        q = ollama.arrays(got, ollama.precision(c0, mode))
        ids, kv = g[f"{name}.ids"].tolist(), ollama.kv_cache(c0, 32)
        out = ollama.forward(ids[:5], list(range(5)), q, c0, kv)
        assert np.allclose(out[0], g[f"{name}.logits"][0], rtol=1e-9, atol=1e-9)


def test_families_outside_the_decode_path_are_refused_by_name(tmp_path):
    import json
    from ferrite_b200 import checkpoint, llama
    fields, _, _ = MODELS["dense_bfp8"]
    _, raw, _, _ = golden_model("dense_bfp8")
    checkpoint.save(str(tmp_path), llama.model(**fields), raw)
    cfg = json.load(open(tmp_path / "config.json")) | {"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}
    json.dump(cfg, open(tmp_path / "config.json", "w"))
    with pytest.raises(AssertionError, match="not covered"):
        checkpoint.load(str(tmp_path))
