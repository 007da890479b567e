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


def test_rows_and_places_outside_the_cache_touch_nothing(cuda):
    # a cache row past the cache (decoding beyond a sequence's part) is not written, a place past the RoPE tables reads
    # the tables' last row, and attention reads no key past the cache whatever a place says: the cache sits inside a
    # larger buffer of a known pattern, which must come back unchanged, and attention equals the clamped oracle
    H, KV, hd, size = 4, 2, 64, 64
    rng = np.random.default_rng(9)
    c = llama.model(dim=H * hd, heads=H, kv=KV, head_dim=hd, layers=1, eps=1e-6, theta=10000.0)
    cos, sin = llama.rotary(c, size)
    guard = 4096
    buf = torch.full((guard + 2 * KV * size * hd + guard,), 7.0, dtype=torch.bfloat16, device=cuda)
    cache = buf[guard:guard + 2 * KV * size * hd].view(2 * KV, size, hd)
    cache.zero_()
    qkv = bfp.bf16_round(rng.normal(0, 1, (3, (H + 2 * KV) * hd)).astype(np.float32))
    places = torch.tensor([5, size + 40, -3], dtype=torch.int32, device=cuda)      # one inside the tables, two outside
    rows = torch.tensor([5, size, -1], dtype=torch.int32, device=cuda)             # one inside the cache, two outside
    ops.rope_kv_write(to_bf16_tensor(qkv, cuda), to_bf16_tensor(cos[:, :hd], cuda).contiguous(), to_bf16_tensor(sin[:, :hd], cuda).contiguous(),
                      places, rows, cache, H, KV, hd)
    torch.cuda.synchronize()
    assert bool((buf[:guard] == 7.0).all()) and bool((buf[-guard:] == 7.0).all()), "nothing outside the cache is written"
    written = to_numpy(cache).any(-1)
    assert written[:, 5].all() and written.sum() == 2 * KV, "only the row inside the cache is written"
    # attention: a place of 10 * size sees the whole cache and nothing more
    cache.copy_(to_bf16_tensor(bfp.bf16_round(rng.normal(0, 1, (2 * KV, size, hd)).astype(np.float32)), cuda))
    q = bfp.bf16_round(rng.normal(0, 1, (2, H * hd)).astype(np.float32))
    base = torch.tensor([0, 32], dtype=torch.int32, device=cuda)
    far = torch.tensor([10 * size, 10 * size], dtype=torch.int32, device=cuda)
    got = to_numpy(ops.decode_attention(to_bf16_tensor(q, cuda), cache, base, far, H, KV, hd, max_keys=size))
    want = attention_oracle(q.astype(np.float64), to_numpy(cache), [0, 32], [size - 1, size - 33], H, KV, hd)
    assert np.abs(got - want).max() < 0.01 * np.abs(want).max() + 1e-3


def test_a_recorded_step_survives_a_larger_workspace(cuda):
    # a step recorded as a CUDA graph holds the address of the attention scratch it was given; a later, larger call
    # replaces that scratch, and the recorded step must still compute what it computed (the replaced buffer stays alive)
    H, KV, hd, size, T = 8, 2, 128, 1024, 4
    gen = torch.Generator(device=cuda).manual_seed(2)
    cache = torch.empty(2 * KV, T * size, hd, dtype=torch.bfloat16, device=cuda).normal_(0, 1, generator=gen)
    q = torch.empty(T, H * hd, dtype=torch.bfloat16, device=cuda).normal_(0, 1, generator=gen)
    base = torch.arange(T, dtype=torch.int32, device=cuda) * size
    place = torch.full((T,), size - 1, dtype=torch.int32, device=cuda)
    out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=cuda)
    ops._ATT_WS.pop(cuda, None)  # start from no scratch, so that the recorded call's is small
    ops.decode_attention(q, cache, base, place, H, KV, hd, size, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.decode_attention(q, cache, base, place, H, KV, hd, size, out=out)
    graph.replay()
    torch.cuda.synchronize()
    want = out.clone()
    held = ops._ATT_WS[cuda]
    # a much larger call: more tokens, so more partial sums than the recorded call's scratch holds
    T2 = 512
    big = ops.attention_workspace(cuda, held.numel() * 4)
    assert big is not held and any(r is held for r in ops._RETIRED), "the replaced scratch is kept"
    fill = torch.empty(64 << 20, dtype=torch.uint8, device=cuda).fill_(255)  # memory a freed scratch would have been handed out as
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want) and int(fill[0]) == 255
