"""Parity at the sizes the benchmark's numbers are quoted on: the isolated matmul grid (K = 4096, N in {4096, 14336},
1..256 rows, both formats, RMSNorm + SwiGLU fused), and one block plus output layer in the Llama-3.1-8B, Mixtral-8x7B
and Qwen3-30B-A3B shapes at their batch sizes and contexts - against the numpy oracle on the same seeded inputs, the way
the reference checks its own 8B shapes (test/test_sim.py:1926-1949: same greedy token, logits within 2 % of their span).

Weights are drawn on the GPU (bf16 values), read back, and quantised for the oracle by the C restatement of the
reference's block-float model, so the two sides share the inputs and nothing else."""
import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor, to_numpy
from ferrite_b200 import ops
from oracle import bfp
from oracle import build as obuild
from oracle import llama as ollama

pytestmark = pytest.mark.gpu

TOL = 0.02  # of the logits' span (test/test_sim.py:1949)


def drawn(cuda, gen, shape, sigma=0.02):
    """N(0, sigma) rounded to bf16 on the device, and the same values as float32 on the host."""
    t = torch.empty(*shape, dtype=torch.float32, device=cuda).normal_(0, sigma, generator=gen).bfloat16()
    return t, t.float().cpu().numpy()


def rel_err(got, want):
    return np.abs(got - want).max() / np.abs(want).max()


@pytest.fixture(scope="module")
def grid_weights(cuda):
    """(fmt, N) -> (packed on the device, float64 values the oracle quantised) for K = 4096."""
    made = {}

    def get(fmt, N):
        if (fmt, N) not in made:
            made.clear()  # one matrix at a time: 4096 x 14336 doubles are 470 MB
            gen = torch.Generator(device=cuda).manual_seed(N + len(fmt))
            t, host = drawn(cuda, gen, (4096, N))
            made[fmt, N] = (ops.quantize(t, fmt), obuild.bfp_values(host, fmt).astype(np.float64))
        return made[fmt, N]
    return get


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("N", [4096, 14336])
def test_matmul_grid_with_norm_and_swiglu(cuda, grid_weights, fmt, N):
    # the isolated-matmul sweep's shapes by the kernel fb_linear picks for each: one row (GEMV), 8 (register-fed MMA or
    # tcgen05), 32 and 128 (tcgen05: one and two activation slots), 129 and 256 (more than one pass of 128 rows)
    K = 4096
    packed, wq = grid_weights(fmt, N)
    rng = np.random.default_rng(N)
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, K)).astype(np.float32))
    for M in (1, 8, 32, 128, 129, 256):
        x = bfp.bf16_round(rng.normal(0, 1, (M, K)).astype(np.float32))
        gu = ollama.rms(x.astype(np.float64), g, 1e-5) @ wq
        want = ollama.glu(gu[:, :N // 2], gu[:, N // 2:])
        tx, tg = to_bf16_tensor(x, cuda), to_bf16_tensor(g, cuda)
        got = to_numpy(ops.linear(tx, packed, norm_w=tg, eps=1e-5, epilogue="swiglu"))
        assert got.shape == (M, N // 2) and rel_err(got, want) < 6e-3, (fmt, N, M, rel_err(got, want))
        plain = to_numpy(ops.linear(tx, packed, norm_w=tg, eps=1e-5, out_dtype="fp32"))
        assert rel_err(plain, gu) < (2e-5 if M == 1 else 4e-3), (fmt, N, M, rel_err(plain, gu))
        # row by row as well: no row of a later pass may be another pass's (each within the bound of its own scale)
        worst = (np.abs(plain - gu).max(1) / np.abs(gu).max(1)).max()
        assert worst < 8e-3, (fmt, N, M, worst)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_residual_epilogue_at_128_rows(cuda, grid_weights, fmt):
    K = N = 4096
    packed, wq = grid_weights(fmt, N)
    rng = np.random.default_rng(11)
    for M in (128, 200):
        x = bfp.bf16_round(rng.normal(0, 1, (M, K)).astype(np.float32))
        r = bfp.bf16_round(rng.normal(0, 1, (M, N)).astype(np.float32))
        want = r + x.astype(np.float64) @ wq
        got32 = to_numpy(ops.linear(to_bf16_tensor(x, cuda), packed, epilogue="residual", residual=to_bf16_tensor(r, cuda), out_dtype="fp32"))
        assert rel_err(got32, want) < 2e-5, (fmt, M, rel_err(got32, want))
        got = to_numpy(ops.linear(to_bf16_tensor(x, cuda), packed, epilogue="residual", residual=to_bf16_tensor(r, cuda)))
        assert rel_err(got, want) < 5e-3


# ---------------------------------------------------------------- one block + output layer at the models' real sizes

@pytest.fixture(scope="module")
def rt(cuda):
    from ferrite_b200.tensor import Runtime
    return Runtime(0)


def block_case(rt, cuda, c, mode, sequences, part, seed):
    """A one-block model in c's shapes on the device and for the oracle: (device weights, oracle weights, device cache,
    oracle cache), the cache of `sequences` parts of `part` rows filled with N(0, 1) bf16 values."""
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    gen = torch.Generator(device=cuda).manual_seed(seed)
    prec = llama.precision(c, mode)
    hd, d, nh = llama.head(c), c.dim, c.heads + 2 * c.kv
    shapes = {"layers.0.qkv_proj": (d, nh * hd), "layers.0.o_proj": (c.heads * hd, d)}
    if c.experts:
        shapes |= {"layers.0.router": (d, c.experts), "layers.0.experts.gate_up": (c.experts, d, 2 * c.moe), "layers.0.experts.down": (c.experts, c.moe, d)}
    else:
        shapes |= {"layers.0.gate_up_proj": (d, 2 * c.ffn), "layers.0.down_proj": (c.ffn, d)}
    shapes |= {"embed": (c.vocab, d)}
    dev, host = {}, {}
    for name, shape in shapes.items():
        t, a = drawn(cuda, gen, shape)
        f = llama.weight_format(name, prec)
        shape3 = (1,) * (3 - t.dim()) + tuple(t.shape)
        x = Tensor(rt, shape3[1], shape3[2], batch=shape3[0], buf=t.view(shape3))
        dev[name] = x.cast(f).realize() if f != "bf16" else x
        host[name] = obuild.bfp_values(a, f) if f != "bf16" else a
        if name == "embed":
            f = llama.weight_format("embed.T", prec)
            tt = t.t().contiguous()
            xt = Tensor(rt, d, c.vocab, buf=tt.view(1, d, c.vocab))
            dev["embed.T"] = xt.cast(f).realize() if f != "bf16" else xt
            host["embed.T"] = obuild.bfp_values(np.ascontiguousarray(a.T), f) if f != "bf16" else np.ascontiguousarray(a.T)
    rng = np.random.default_rng(seed)
    norms = {k: bfp.bf16_round(rng.normal(1, 0.1, (1, d)).astype(np.float32)) for k in ("layers.0.input_layernorm", "layers.0.post_attention_layernorm", "norm")}
    if c.qk_norm:
        qn, kn = (bfp.bf16_round(rng.normal(1, 0.1, (1, hd)).astype(np.float32)) for _ in range(2))
        norms["layers.0.qk_norm"] = np.stack([qn] * c.heads + [kn] * c.kv)
        host["layers.0.qk_on"] = np.array([1.0] * (c.heads + c.kv) + [0.0] * c.kv, np.float32).reshape(nh, 1, 1)
    for k, a in norms.items():
        dev[k] = Tensor.of(rt, a)
        host[k] = a if k != "layers.0.qk_norm" else np.concatenate([a, np.ones((c.kv, 1, hd), np.float32)])
    cos, sin = llama.rotary(c, c.places)
    dev["cos"], dev["sin"] = Tensor.of(rt, cos), Tensor.of(rt, sin)
    host["cos"], host["sin"] = ollama.rotary(c, c.places)
    kv = Tensor(rt, sequences * part, hd, batch=2 * c.kv)
    kv.buf.normal_(0, 1, generator=gen)
    return dev, host, [kv], [kv.buf.float().cpu().numpy()]


def check_rows(got, want, what):
    for u in range(len(want)):
        span, err = np.ptp(want[u]), np.abs(got[u] - want[u]).max()
        top2 = np.sort(want[u])[-2:]
        assert err <= TOL * span, (what, u, err / span)
        assert got[u].argmax() == want[u].argmax() or top2[1] - top2[0] <= 2 * err, (what, u, err / span)


def test_llama_8b_shape_block_32_sequences_at_2048(rt, cuda):
    # the benchmark's workload, one block of it: 32 sequences decoding together at places 2048.. over a cache of N(0, 1)
    # keys and values, then the output layer over a quarter of the vocabulary (a 4-rank shard; 131 M values)
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor, jit
    S, part = 32, 2112
    kw = dict(dim=4096, heads=32, kv=8, layers=1, vocab=32064, ffn=14336, theta=500000.0, eps=1e-5, places=part)
    c, oc = llama.model(**kw), ollama.model(**kw)
    dev, host, kv, okv = block_case(rt, cuda, c, "bfp8", S, part, seed=3)
    rng = np.random.default_rng(3)
    on = lambda row: Tensor.of(rt, [row], "int32")
    step = jit(lambda ids, places: llama.forward(ids, places, dev, c, kv, S))
    for i in range(3):  # eager, recorded, replayed
        ids, places = rng.integers(0, c.vocab, S).tolist(), [2048 + i] * S
        got = step(on(ids), on(places)).numpy()[0]
        want = ollama.forward(ids, places, host, oc, okv, S)
        check_rows(got, want, ("8b", i))
    # the keys and values the steps wrote are the oracle's, to a bf16 rounding
    row = 5 * part + 2049
    assert rel_err(kv[0].buf[:, row].float().cpu().numpy(), okv[0][:, row]) < 1e-2


def test_mixtral_shape_block_64_sequences_at_1024(rt, cuda):
    # top-2 of 8 experts of 14336 in bfp4, attention and output layer in bfp8, 64 sequences at context 1024
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    S, part = 64, 1088
    kw = dict(dim=4096, heads=32, kv=8, layers=1, vocab=4096, ffn=0, experts=8, k=2, moe=14336, norm_topk=True, theta=1000000.0, eps=1e-5, places=part)
    c, oc = llama.model(**kw), ollama.model(**kw, by_expert=True)
    dev, host, kv, okv = block_case(rt, cuda, c, "experts", S, part, seed=4)
    assert dev["layers.0.experts.gate_up"].dtype == "bfp4" and dev["layers.0.qkv_proj"].dtype == "bfp8"
    rng = np.random.default_rng(4)
    on = lambda row: Tensor.of(rt, [row], "int32")
    ids, places = rng.integers(0, c.vocab, S).tolist(), [1024] * S
    picks = device_picks(rt, dev, host, c, oc, kv, okv, ids, places, S)
    got = llama.forward(on(ids), on(places), dev, c, kv, S).numpy()[0]
    want = ollama.forward(ids, places, host, oc, okv, S, picks=[picks])
    check_rows(got, want, "mixtral")
    router_ids_follow_numpy(rt, dev, host, oc, S, rng)


def test_qwen3_shape_block_128_sessions_ragged(rt, cuda):
    # top-8 of 128 experts of 768, QK-norm, 128 sessions whose contexts differ (ragged places), all bfp8
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    S, part = 128, 2048
    kw = dict(dim=2048, heads=32, kv=4, head_dim=128, layers=1, vocab=4096, ffn=0, experts=128, k=8, moe=768, norm_topk=True, qk_norm=True,
              theta=1000000.0, eps=1e-6, places=part)
    c, oc = llama.model(**kw), ollama.model(**kw, by_expert=True)
    dev, host, kv, okv = block_case(rt, cuda, c, "bfp8", S, part, seed=6)
    rng = np.random.default_rng(6)
    on = lambda row: Tensor.of(rt, [row], "int32")
    ids, places = rng.integers(0, c.vocab, S).tolist(), rng.integers(64, part - 2, S).tolist()
    picks = device_picks(rt, dev, host, c, oc, kv, okv, ids, places, S)
    got = llama.forward(on(ids), on(places), dev, c, kv, S).numpy()[0]
    want = ollama.forward(ids, places, host, oc, okv, S, picks=[picks])
    check_rows(got, want, "qwen3")
    router_ids_follow_numpy(rt, dev, host, oc, S, rng)


def device_picks(rt, dev, host, c, oc, kv, okv, ids, places, S):
    """The experts the device's router picks for the block's tokens: the block's first half run piece by piece on the
    device (embedding, attention, RMSNorm, router logits in fp32, top-k).  They must be numpy's stable top-k of those
    very logits, bit for bit, and the oracle's own picks wherever the oracle's k-th logit stands clear of the next (by
    1 % of the row's span: the hidden state the device routes is rounded to bf16); the oracle then runs the device's
    picks, so that a near tie does not compare two different sets of experts."""
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Tensor
    on = lambda row: Tensor.of(rt, [row], "int32")
    p = llama.block(dev, "layers.0.")
    x = dev["embed"].gather(on(ids))
    rows, seen, _ = llama.around(dev, c, on(places), kv[0].rows, S)
    x = llama.added(x, llama.attention(llama.rms(x, p["input_layernorm"], c), p, c, (dev["cos"], dev["sin"], on(places)), seen, kv[0], rows, S), c).realize()
    logits = llama.rms(x, p["post_attention_layernorm"], c).matmul(p["router"], dtype="fp32").realize()
    _, picked = logits.topk(c.k)
    stored, picked = logits.numpy()[0], picked.numpy()[0]
    assert np.array_equal(picked, ollama.topk(stored, c.k)[1]), "the picks are the stable top-k of the stored logits"
    # the oracle's logits for the same tokens (its cache rows for this step are written by this call too)
    op = ollama.block(host, "layers.0.")
    ox = host["embed"][list(ids)].astype(np.float64)
    orows, cos, sin, mask, _ = ollama.around(host, oc, places, okv[0].shape[-2], S)
    ox = ox + ollama.attention(ollama.rms(ox, op["input_layernorm"], oc.eps), op, oc, cos, sin, mask, okv[0], orows, S)
    exact = ollama.rms(ox, op["post_attention_layernorm"], oc.eps) @ op["router"]
    assert np.abs(stored - exact).max() < 0.01 * np.ptp(exact), "router logits"
    ranked = np.sort(exact, -1)[:, ::-1]
    clear = (ranked[:, c.k - 1] - ranked[:, c.k]) > 0.01 * np.ptp(exact, -1)
    same = np.array([set(a) == set(b) for a, b in zip(picked, ollama.topk(exact, c.k)[1])])
    assert same[clear].all(), "where the oracle's k-th logit stands clear of the next, the device picks the oracle's experts"
    return picked


def router_ids_follow_numpy(rt, dev, host, oc, S, rng):
    """The device's picks are numpy's stable top-k of the device's own router logits, bit for bit (the order of
    models/llama.py:27), and its softmax weights those of the picked values (models/llama.py:287-288)."""
    from ferrite_b200.tensor import Tensor
    h = bfp.bf16_round(rng.normal(0, 1, (S, oc.dim)).astype(np.float32))
    logits = Tensor.of(rt, h).matmul(dev["layers.0.router"], dtype="fp32").realize()
    values, ids = logits.topk(oc.k)
    stored = logits.numpy()[0]
    want_values, want_ids = ollama.topk(stored, oc.k)
    assert np.array_equal(ids.numpy()[0], want_ids) and np.array_equal(values.numpy()[0], want_values)
    exact = h.astype(np.float64) @ host["layers.0.router"]
    assert np.abs(stored - exact).max() < 2e-5 * np.abs(exact).max()
