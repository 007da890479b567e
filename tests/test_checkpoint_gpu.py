"""The checkpoint reader's device side: every weight assembled on the GPU (pieces uploaded as they lie in the file,
transposed and joined by the strided copy kernel) equals the host recipe bit for bit, and the model uploaded from the
file - cast to block float on the device - decodes the golden logits (the reference's load -> upload -> forward,
models/llama.py:572-604, 628-640)."""
import numpy as np
import pytest

from conftest import golden
from test_llama_gpu import agrees
from test_oracle import MODELS, golden_model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("dense_bfp8", "BF16"), ("dense_bfp4", "F32"), ("moe_top2", "BF16")])
def test_model_from_a_checkpoint_decodes(cuda, tmp_path, name, dtype):
    from ferrite_b200 import checkpoint, llama
    from ferrite_b200.tensor import Runtime, Tensor
    rt = Runtime(0)
    fields, mode, _ = MODELS[name]
    _, raw, _, _ = golden_model(name)
    checkpoint.save(str(tmp_path), llama.model(**fields), raw, dtype, shards=2)
    c, w = checkpoint.load(str(tmp_path), places=64)
    for k in ("layers.0.qkv_proj", "layers.1.o_proj", "embed.T", "norm") + (("layers.0.experts.gate_up", "layers.1.router") if c.experts else ("layers.1.gate_up_proj",)):
        dev = w[k].device(rt)
        assert np.array_equal(dev.numpy().reshape(w[k].values().shape), w[k].values()), k
    t = llama.upload(rt, w, llama.precision(c, mode))
    assert t["layers.0.qkv_proj"].dtype == "bfp8" and t["embed"].dtype == "bf16"
    g = golden("models.npz")
    kv = llama.kv_cache(c, 32, llama.zeros(rt))
    on = lambda row: Tensor.of(rt, [row], "int32")
    ids, want = g[f"{name}.ids"].tolist(), g[f"{name}.logits"]
    for i in range(3):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        ok, detail = agrees(llama.logits(llama.forward(on(new), on(places), t, c, kv)), want[i])
        assert ok, (name, i, detail)
