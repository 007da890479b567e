"""A block-float KV cache (bfp8 / bfp4), after the reference's test of it (test/test_sim.py:2081-2107): rows written
into it are rounded run by run exactly as the cast rounds them (numpy's bfp, bit for bit), and attention over it is bit
for bit attention over a bf16 cache holding the same values; then a whole decoder with such a cache against the numpy
restatement that rounds what it caches."""
import numpy as np
import pytest
import torch

from oracle import bfp
from oracle import llama as ollama

pytestmark = pytest.mark.gpu


def bf16_tensor(a, device):
    return torch.from_numpy(bfp.bf16_round(np.asarray(a, np.float32))).to(device).bfloat16()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("hd", [64, 128])
def test_put_rounds_like_the_cast_and_attention_reads_it_in_place(cuda, fmt, hd):
    from ferrite_b200 import ops
    rng = np.random.default_rng(16)
    H, KV, size, T = 8, 2, 192, 3
    cache = ops.Packed(fmt, 2 * KV, size, hd, torch.zeros(2 * KV * ops.lib().fb_packed_bytes(ops._lib.DTYPES[fmt], size, hd), dtype=torch.uint8, device=cuda))
    want = np.zeros((2 * KV, size, hd), np.float32)
    ones, zeros = bf16_tensor(np.ones((256, hd)), cuda), bf16_tensor(np.zeros((256, hd)), cuda)  # tables that turn nothing
    for rows in ([5, 70, 191], [0, 64, 128], [63, 65, 127]):
        x = bfp.bf16_round((rng.normal(0, 2, (T, (H + 2 * KV) * hd)) * 10.0 ** rng.integers(-3, 3, (T, 1))).astype(np.float32))
        places = torch.zeros(T, dtype=torch.int32, device=cuda)
        ops.rope_kv_write(bf16_tensor(x, cuda), ones, zeros, places, torch.tensor(rows, dtype=torch.int32, device=cuda), cache, H, KV, hd)
        kv = x.reshape(T, H + 2 * KV, hd)[:, H:].transpose(1, 0, 2)  # [2KV, T, hd]
        want[:, rows] = bfp.bfp(kv, fmt)
        got = ops.dequantize(cache).float().cpu().numpy()
        assert np.array_equal(got, want), (fmt, hd, rows)
    # attention over the packed cache == attention over a bf16 cache of the same values, bit for bit
    full = bfp.bfp(rng.normal(0, 1, (2 * KV, size, hd)).astype(np.float32), fmt)
    same = bf16_tensor(full, cuda)
    packed = ops.quantize(same, fmt)
    assert np.array_equal(ops.dequantize(packed).float().cpu().numpy(), full)
    q = bf16_tensor(rng.normal(0, 1, (T, H * hd)), cuda)
    base = torch.tensor([0, 64, 0], dtype=torch.int32, device=cuda)
    for place, window in (([190, 100, 3], 0), ([63, 64, 127], 0), ([150, 120, 80], 70)):
        last = torch.tensor(place, dtype=torch.int32, device=cuda)
        a = ops.decode_attention(q, packed, base, last, H, KV, hd, size, window=window)
        b = ops.decode_attention(q, same, base, last, H, KV, hd, size, window=window)
        assert torch.equal(a, b), (fmt, hd, place, window)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_decoder_with_a_block_float_cache(cuda, fmt):
    """A prompt and four decode steps with the cache in block float against the REFERENCE's logits for the same
    (tests/golden/kv.npz, made by the reference's numpy branch, which rounds what it caches): within 2 % of the logits'
    span, as the bf16-cache decoders are held to; and the cache itself against the restatement's."""
    import copy

    from conftest import golden
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Runtime, Tensor
    from test_oracle import golden_model
    rt, g = Runtime(0), golden("kv.npz")
    c, raw, arrays, _ = golden_model("dense_bfp8")
    oc = copy.copy(c)
    oc.cache = fmt
    kv_o = ollama.kv_cache(oc, 64)
    t = llama.upload(rt, raw, llama.precision(c, "bfp8"))
    kv_d = llama.kv_cache(c, 64, llama.zeros(rt, fmt))
    assert kv_d[0].dtype == fmt
    on = lambda row: Tensor.of(rt, [row], "int32")
    ids, want = g[f"{fmt}.ids"].tolist(), g[f"{fmt}.logits"]
    for i in range(5):
        new = ids[:5] if i == 0 else ids[4 + i:5 + i]
        places = list(range(5)) if i == 0 else [4 + i]
        got = llama.logits(llama.forward(on(new), on(places), t, c, kv_d))
        ollama.forward(new, places, arrays, oc, kv_o)
        assert np.abs(got - want[i]).max() <= 0.02 * np.ptp(want[i]), (fmt, i)
    # what the device cached is what numpy's rounded cache holds, up to one step of the format where the activations'
    # bf16 rounding on the device tips a value over a rounding boundary
    step = {"bfp8": 0.02, "bfp4": 0.2}[fmt]
    for l in range(c.layers):
        dev, ref = kv_d[l].numpy()[:, :9], kv_o[l][:, :9]
        assert np.abs(dev - ref).max() <= step * np.abs(ref).max(), l
