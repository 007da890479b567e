"""RoPE + KV write, decode attention, gather, RMSNorm, argmax against the numpy oracle
(the numpy halves of the reference's test_attend / test_put / test_llama_layer, test/test_sim.py:641-680, 2063-2079)."""
import math

import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor, to_numpy
from ferrite_b200 import ops
from oracle import bfp, llama

pytestmark = pytest.mark.gpu


def test_gather_and_argmax_and_rmsnorm(cuda):
    rng = np.random.default_rng(1)
    table = bfp.bf16_round(rng.normal(0, 1, (300, 576)).astype(np.float32))
    ids = rng.integers(0, 300, 40)
    got = ops.gather_rows(to_bf16_tensor(table, cuda), torch.tensor(ids, dtype=torch.int32, device=cuda))
    assert np.array_equal(to_numpy(got), table[ids])
    logits = rng.normal(0, 3, (5, 49152)).astype(np.float32)
    logits[2, 700] = logits[2, 41000] = logits[2].max() + 1  # a tie: the lower column wins, as numpy's argmax
    assert to_numpy(ops.argmax(torch.tensor(logits, device=cuda))).tolist() == logits.argmax(-1).tolist()
    x, w = bfp.bf16_round(rng.normal(0, 2, (7, 576)).astype(np.float32)), bfp.bf16_round(rng.normal(1, 0.1, (1, 576)).astype(np.float32))
    want = llama.rms(x.astype(np.float64), w, 1e-5)
    got = to_numpy(ops.rmsnorm(to_bf16_tensor(x, cuda), to_bf16_tensor(w, cuda), 1e-5))
    assert np.abs(got - want).max() < 2 ** -8 * np.abs(want).max()


@pytest.mark.parametrize("H,KV,hd,qk", [(9, 3, 64, False), (32, 8, 128, False), (4, 2, 128, True)])
@pytest.mark.parametrize("wide", [False, True])
def test_rope_and_cache_write(cuda, H, KV, hd, qk, wide):
    rng = np.random.default_rng(H + hd)
    c = llama.model(dim=H * hd, heads=H, kv=KV, head_dim=hd, layers=1, eps=1e-6, theta=10000.0)
    T, size, nh = 6, 64, H + 2 * KV
    cos, sin = llama.rotary(c, size)  # [size, nh*hd]
    qkv = bfp.bf16_round(rng.normal(0, 1, (T, nh * hd)).astype(np.float32))
    places, rows = rng.integers(0, size, T), rng.permutation(size)[:T]
    norm = bfp.bf16_round(rng.normal(1, 0.2, (H + KV, hd)).astype(np.float32)) if qk else None
    heads = llama.split_heads(qkv.astype(np.float64), nh)
    if qk:
        r = 1 / np.sqrt((heads * heads).mean(-1, keepdims=True) + c.eps)
        scale = np.concatenate([norm[:, None, :], np.ones((KV, 1, hd))], 0)
        on = np.array([1.0] * (H + KV) + [0.0] * KV).reshape(nh, 1, 1)
        heads = heads * np.where(on, r * scale, 1)
    want = heads * llama.split_heads(cos[places].astype(np.float64), nh) + llama.rotate_half(heads) * llama.split_heads(sin[places].astype(np.float64), nh)
    cache = torch.zeros(2 * KV, size, hd, dtype=torch.bfloat16, device=cuda)
    tcos, tsin = (to_bf16_tensor(t if wide else t[:, :hd], cuda).contiguous() for t in (cos, sin))
    q = ops.rope_kv_write(to_bf16_tensor(qkv, cuda), tcos, tsin, torch.tensor(places, dtype=torch.int32, device=cuda),
                          torch.tensor(rows, dtype=torch.int32, device=cuda), cache, H, KV, hd,
                          qk_norm=to_bf16_tensor(norm, cuda) if qk else None, eps=c.eps)
    tol = 2 ** -8 * 4
    assert np.abs(to_numpy(q) - llama.merge_heads(want[:H])).max() < tol
    got = to_numpy(cache)
    assert np.abs(got[:, rows] - want[H:]).max() < tol
    untouched = np.ones(size, bool); untouched[rows] = False
    assert not got[:, untouched].any(), "only the tokens' rows are written"


def attention_oracle(q, cache, base, place, H, KV, hd, window=0):
    T, rep, out = q.shape[0], H // KV, np.zeros((q.shape[0], H * hd))
    for t in range(T):
        first = max(0, place[t] + 1 - window) if window else 0
        keys = slice(base[t] + first, base[t] + place[t] + 1)
        for h in range(H):
            k, v = cache[h // rep, keys], cache[KV + h // rep, keys]
            s = k @ q[t, h * hd:(h + 1) * hd] / math.sqrt(hd)
            p = np.exp(s - s.max())
            out[t, h * hd:(h + 1) * hd] = (p / p.sum()) @ v
    return out


@pytest.mark.parametrize("T,H,KV,hd,size,window", [(1, 9, 3, 64, 96, 0), (4, 32, 8, 128, 2200, 0), (32, 32, 8, 128, 320, 0),
                                                   (3, 32, 4, 128, 700, 0), (2, 8, 8, 64, 300, 50), (5, 4, 2, 128, 33, 0)])
def test_decode_attention(cuda, T, H, KV, hd, size, window):
    rng = np.random.default_rng(T * 100 + size)
    cache = bfp.bf16_round(rng.normal(0, 1, (2 * KV, T * size, hd)).astype(np.float32))
    q = bfp.bf16_round(rng.normal(0, 1, (T, H * hd)).astype(np.float32))
    base = np.arange(T) * size
    place = rng.integers(0, size, T)
    place[0], place[-1] = size - 1, 0 if T > 1 else size - 1  # the longest and the shortest
    want = attention_oracle(q.astype(np.float64), cache.astype(np.float64), base, place, H, KV, hd, window)
    got = to_numpy(ops.decode_attention(to_bf16_tensor(q, cuda), to_bf16_tensor(cache, cuda), torch.tensor(base, dtype=torch.int32, device=cuda),
                                        torch.tensor(place, dtype=torch.int32, device=cuda), H, KV, hd, max_keys=size, window=window))
    assert np.abs(got - want).max() < 0.01 * np.abs(want).max() + 1e-3, np.abs(got - want).max()  # the reference's own bound: 1% (test_sim.py:674)


def test_attention_misuse_is_refused(cuda):
    q = torch.zeros(1, 96, dtype=torch.bfloat16, device=cuda)
    cache = torch.zeros(2, 32, 96, dtype=torch.bfloat16, device=cuda)
    z = torch.zeros(1, dtype=torch.int32, device=cuda)
    with pytest.raises(AssertionError):
        ops.decode_attention(q, cache, z, z, 1, 1, 96, max_keys=32)  # heads are 64 or 128 wide
