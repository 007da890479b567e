"""Llama-family decoder in numpy: the CPU restatement the CUDA path is checked against.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Restates the numpy branch of the
reference's models/llama.py (the branch `fns` picks for np.ndarray, llama.py:26-39) and
the helpers it borrows from models/gpt2.py.  The dtype flow is the reference's: float32
weights, np.zeros (float64) KV caches, exact products, no bf16 rounding of activations.
Each function names the reference lines it follows.
"""
import math
from types import SimpleNamespace

import numpy as np

from . import bfp as _bfp

# config fields beyond a plain Llama's, with a plain Llama's values (models/llama.py:541-543)
_DEFAULTS = dict(head_dim=None, rope=None, k=0, experts=0, moe=0, norm_topk=True, tied=False, precision=None,
                 places=4096, ffn=None, vocab=None, qk_norm=False)


def model(**fields):
    """A config object: dim, heads, kv, layers, eps, theta, vocab, ffn (+ the MoE and Qwen3 extras)."""
    return SimpleNamespace(**(_DEFAULTS | fields))


def head(c):
    """Width of one attention head (models/llama.py:87)."""
    return c.head_dim or c.dim // c.heads


# ---------------------------------------------------------------- formats

def precision(c, mode="bf16"):
    """{(op, block): format} for the weight matrices (the format half of models/llama.py:54-76).

    bf16 / bfp8: everything in that format; bfp4: gate_up in bfp4 and the rest bfp8;
    experts: gate_up and down (the experts') in bfp4, the rest bfp8.
    """
    four = {"bfp4": ("gate_up",), "experts": ("gate_up", "down")}.get(mode, ())

    def fmt(op):
        if mode in ("bf16", "bfp8"):
            return mode
        return "bfp4" if op in four else "bfp8"

    table = {(op, l): fmt(op) for l in range(c.layers) for op in ("qkv", "o", "gate_up", "down")}
    table["head", None] = fmt("head")
    return table


def weight_format(name, prec):
    """Format of the weight called `name` (models/llama.py:615-623): matrices a matmul reads as its B
    take the precision table's entry, everything else stays bf16."""
    if not prec:
        return "bf16"
    if name == "embed.T":
        return prec.get(("head", None), "bf16")
    if name.startswith("layers.") and name.endswith(("_proj", "experts.gate_up", "experts.down")):
        op = name.split(".")[-1].removesuffix("_proj")
        return prec.get((op, int(name.split(".")[1])), "bf16")
    return "bf16"


def arrays(weights, prec=None):
    """name -> float32 array as the device holds it: block-float matrices rounded by the bfp model
    (models/llama.py:645-654), made once."""
    out = {}
    for name, w in weights.items():
        f = weight_format(name, prec)
        w = np.asarray(w, np.float32)
        out[name] = w if f == "bf16" else _bfp.bfp_f32(w, f)
    return out


# ---------------------------------------------------------------- pieces of a block

def rms(x, w, eps):
    """RMSNorm scaled by w (models/llama.py:82-85)."""
    return x * (1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)) * w


def frequencies(c):
    """RoPE inverse frequencies in float32, optionally with Llama-3 scaling (models/llama.py:333-349)."""
    hd = head(c)
    inv = 1 / c.theta ** (np.arange(0, hd, 2, dtype=np.float32) / hd)
    r = c.rope
    if r and r.get("rope_type") == "llama3":
        old = r["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        scaled = np.where(wavelen > old / r["low_freq_factor"], inv / r["factor"], inv)
        smooth = (old / wavelen - r["low_freq_factor"]) / (r["high_freq_factor"] - r["low_freq_factor"])
        between = (wavelen >= old / r["high_freq_factor"]) & (wavelen <= old / r["low_freq_factor"])
        inv = np.where(between, (1 - smooth) * scaled / r["factor"] + smooth * scaled, scaled).astype(np.float32)
    return inv


def rotary(c, n):
    """cos and sin tables for places 0..n-1: angles in float32, tables rounded to bf16, one head's
    table repeated for every q and k head, and 1 / 0 for the v heads (models/llama.py:351-368).
    Shapes [n, (heads + 2 kv) * hd]."""
    hd = head(c)
    angles = np.arange(n, dtype=np.float32)[:, None] * frequencies(c)[None]
    per_head = lambda t: np.concatenate([t, t], 1)  # both halves of a head turn by the same angle
    still = lambda v: np.full((n, hd), v, np.float32)
    wide = lambda t, v: np.concatenate([per_head(t)] * (c.heads + c.kv) + [still(v)] * c.kv, 1)
    return _bfp.bf16_round(wide(np.cos(angles), 1)), _bfp.bf16_round(wide(np.sin(angles), 0))


def rotate_half(x):
    """(-x2, x1) over each head's two halves: what the reference writes as x @ turn (models/llama.py:92-93, 361-362)."""
    half = x.shape[-1] // 2
    return np.concatenate([-x[..., half:], x[..., :half]], -1)


def split_heads(a, n):
    """[tokens, n*w] -> [n, tokens, w] (models/gpt2.py:51)."""
    return a.reshape(a.shape[0], n, -1).transpose(1, 0, 2)


def merge_heads(a):
    """[n, tokens, w] -> [tokens, n*w] (models/gpt2.py:55)."""
    return a.transpose(1, 0, 2).reshape(a.shape[1], -1)


def softmax(a):
    e = np.exp(a - a.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def key_mask(column, width):
    """0 where a query at place column[i] may look at key j <= place, else -1e9 (models/gpt2.py:107-110)."""
    return np.where(np.arange(width) > column, np.float32(-1e9), np.float32(0))


def attention(h, p, c, cos, sin, mask, cache, rows, slots=None):
    """One block's attention over its KV cache (models/llama.py:111-146), numpy branch.

    h: [n, dim]; cos/sin: [n, (H+2KV)*hd] rows of the rotary tables for these tokens;
    cache: [2*KV, size, hd] (keys' heads then values'), written in place at `rows`;
    mask: [n, width] without slots, [KV*slots, (n/slots)*rep, width] with them.
    """
    H, KV, hd = c.heads, c.kv, head(c)
    rep, nh, n = H // KV, H + 2 * KV, h.shape[0]
    qkv = split_heads(h @ p["qkv_proj"], nh)
    if "qk_norm" in p:  # Qwen3: each q and k head RMS-normed before it turns; v's left alone (llama.py:121-123)
        r = 1.0 / np.sqrt((qkv * qkv).mean(-1, keepdims=True) + c.eps)
        qkv = qkv * np.where(p["qk_on"], r * p["qk_norm"], 1)
    qkv = qkv * split_heads(cos, nh) + rotate_half(qkv) * split_heads(sin, nh)
    flat = merge_heads(qkv)
    kv = qkv[H:]  # this call's keys and values, at once; a block-float cache rounds them (llama.py:126-128)
    cache[:, list(rows)] = _bfp.bfp(kv, c.cache) if getattr(c, "cache", "bf16") != "bf16" else kv
    q, k, v = qkv[:H], cache[:KV], cache[KV:]
    if slots:  # a batch entry per (kv head, sequence): its rep query heads' rows side by side (llama.py:132-135)
        t = n // slots
        k = k.reshape(KV * slots, -1, hd)
        v = v.reshape(KV * slots, -1, hd)
        q = split_heads(flat[:, :H * hd], KV).reshape(KV * slots, t * rep, hd)
    width = mask.shape[-1]
    if width < k.shape[-2]:
        k, v = k[:, :width], v[:, :width]
    if not slots:
        k, v = np.repeat(k, rep, 0), np.repeat(v, rep, 0)
    s = q @ k.swapaxes(-1, -2) * (1 / math.sqrt(hd))
    o = softmax(s + mask) @ v
    if slots:
        o = o.reshape(KV, n, rep * hd)
    return merge_heads(o) @ p["o_proj"]


def glu(gate, up):
    """SwiGLU: silu(gate) * up (models/llama.py:271-275, no limit)."""
    return gate / (1 + np.exp(-gate)) * up


def mlp(h, p):
    """silu(h @ gate) * (h @ up) @ down with gate and up side by side in gate_up_proj (models/llama.py:266-269)."""
    m = p["down_proj"].shape[-2]
    gu = h @ p["gate_up_proj"]
    return glu(gu[:, :m], gu[:, m:]) @ p["down_proj"]


def topk(a, k):
    """k largest of each row, largest first, lower column first among equals (models/llama.py:27)."""
    ids = np.argsort(-a, -1, kind="stable")[..., :k]
    return np.take_along_axis(a, ids, -1), ids


def experts(h, p, ids, w):
    """Each token's chosen experts' SwiGLUs, weighted and summed (models/llama.py:294-300)."""
    gu, down = p["experts.gate_up"], p["experts.down"]
    m = down.shape[-2]

    def one(x, e):
        g = x @ gu[e]
        return glu(g[:m], g[m:]) @ down[e]

    rows = []
    for t in range(len(h)):
        terms = [w[t, j] * one(h[t], e) for j, e in enumerate(ids[t])]
        acc = terms[0]
        for term in terms[1:]:
            acc = acc + term
        rows.append(acc)
    return np.stack(rows)


def experts_by_expert(h, p, ids, w):
    """experts(), with each expert's matrices multiplied once by all the tokens that pick it instead of once per token
    and pick (the same terms, added per token in the same order): for mixtures whose experts are too large to widen to
    float64 a hundred times over.  tests/test_oracle.py holds it equal to experts()."""
    gu, down = p["experts.gate_up"], p["experts.down"]
    m = down.shape[-2]
    terms = {}
    for e in sorted({int(v) for v in ids.ravel()}):
        rows = [t for t in range(len(h)) if e in ids[t]]
        g = h[rows] @ gu[e]
        y = glu(g[:, :m], g[:, m:]) @ down[e]
        terms |= {(t, e): y[i] for i, t in enumerate(rows)}
    out = []
    for t in range(len(h)):
        acc = w[t, 0] * terms[t, int(ids[t, 0])]
        for j in range(1, ids.shape[1]):
            acc = acc + w[t, j] * terms[t, int(ids[t, j])]
        out.append(acc)
    return np.stack(out)


def moe(h, p, c, live=None, picks=None):
    """Router logits -> top-k -> softmax weights -> weighted experts (models/llama.py:277-292).
    picks (not in the reference): expert ids [tokens, k] to use instead of this function's own top-k, their weights
    still computed here from this function's logits - a test feeds the device's picks so that a near tie between the
    k-th and the next logit, which a bf16 rounding of the hidden state can turn, does not send the two down different
    experts (the reference's own test picks prompts without such ties instead, test/test_sim.py:1550-1552)."""
    logits = h @ p["router"]
    if picks is not None:
        ids = np.asarray(picks)
        chosen = np.take_along_axis(logits if c.norm_topk else softmax(logits), ids, -1)
        w = softmax(chosen) if c.norm_topk else chosen
    elif c.norm_topk:
        vals, ids = topk(logits, c.k)
        w = softmax(vals)
    else:
        w, ids = topk(softmax(logits), c.k)
    run = experts_by_expert if getattr(c, "by_expert", False) else experts
    return run(h, p, ids, w if live is None else w * live)


def touched(ids, weights, n):
    """What Tensor.touched gives (ferrite/tensor.py:403-416): the experts some row picks with a weight
    that is not 0, ascending, then n (none) up to min(rows*k, n) entries; and for each entry each row's
    weight for that expert (0 where the row did not pick it)."""
    rows, k = ids.shape
    slots = min(rows * k, n)
    picked = sorted({int(e) for e, w in zip(ids.ravel(), weights.ravel()) if w != 0 and e < n})
    listed = (picked + [n] * slots)[:slots]
    out = np.zeros((slots, rows, 1), weights.dtype)
    for s, e in enumerate(listed):
        if e < n:
            hit = (ids == e) & (weights != 0)
            out[s, :, 0] = np.where(hit, weights, 0).sum(-1)
    return np.array(listed, np.int32).reshape(slots, 1), out


def group(ids, n):
    """What Tensor.group gives (ferrite/tensor.py:389-402), after the one-worker kernel that computes it on the chip
    (ferrite/compiler.py:1842-1896): each value's choices counted, its run of slots starting where the runs of the values
    before it end, each rounded up to whole tiles of 32, each choice taking the next slot of its value's run in the
    choices' own order.  (order [32 t], tiles [t], places [k rp]) as int32 arrays."""
    ids = np.asarray(ids)
    rows, k = ids.shape
    t, rp = -(-rows * k // 32) + min(n, rows * k), -(-rows // 32) * 32
    fill = np.bincount(ids.ravel(), minlength=n)[:n].astype(np.int64)
    order, tiles, places = np.zeros(32 * t, np.int32), np.full(t, n, np.int32), np.zeros(k * rp, np.int32)
    s = 0
    for e in range(n):
        count, fill[e] = fill[e], s
        end = s + -(-count // 32) * 32
        tiles[s // 32:end // 32] = e
        s = end
    for r in range(rows):
        for j in range(k):
            s = fill[ids[r, j]]
            fill[ids[r, j]] += 1
            order[s], places[j * rp + r] = r, s
    return order, tiles, places


def block(w, prefix):
    """The weights named prefix..., by the rest of their names (models/gpt2.py:70)."""
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def layer(x, p, c, cos, sin, mask, cache, rows, live=None, slots=None, picks=None):
    """Attention then MLP (or MoE), each after an RMSNorm and added back (models/llama.py:95-109)."""
    x = x + attention(rms(x, p["input_layernorm"], c.eps), p, c, cos, sin, mask, cache, rows, slots)
    h = rms(x, p["post_attention_layernorm"], c.eps)
    return x + (moe(h, p, c, live, picks) if "router" in p else mlp(h, p))


def around(w, c, places, size, slots=None):
    """Cache rows, rotary rows, mask and the live column for tokens at `places` (models/llama.py:429-452)."""
    places = np.asarray(places)
    n = places.shape[-1]
    cos, sin = w["cos"][places], w["sin"][places]
    at = places.reshape(-1, 1)
    if not slots:
        return places, cos, sin, key_mask(at, size), None
    part, rep = size // slots, c.heads // c.kv
    rows = places + np.array([i // (n // slots) * part for i in range(n)])
    live = (at < part - 1).astype(np.float32)  # a free slot's token sits on its part's last row
    seen = np.where(at < part - 1, at, 0)
    column = np.broadcast_to(seen.reshape(1, n, 1), (1, n, rep)).reshape(1, n * rep, 1)
    column = np.broadcast_to(column, (c.kv, n * rep, 1)).reshape(c.kv * slots, n // slots * rep, 1)
    return rows, cos, sin, key_mask(column, part), live


def forward(ids, places, w, c, caches, slots=None, every=False, picks=None):
    """Logits for the token after `ids` at `places` (models/llama.py:459-480): the last token's, or every
    token's with slots / every.  picks: per block, the experts to use (see moe), or None."""
    x = w["embed"][list(ids)]
    size = caches[0].shape[-2]
    rows, cos, sin, mask, live = around(w, c, places, size, slots)
    for l in range(c.layers):
        x = layer(x, block(w, f"layers.{l}."), c, cos, sin, mask, caches[l], rows, live, slots, picks[l] if picks else None)
    h = rms(x, w["norm"], c.eps)
    return (h if slots or every else h[-1:]) @ w["embed.T"]


def prefill(ids, w, c, caches, tokens):
    """forward over a prompt from place 0, `tokens` at a time (models/llama.py:498-504); the logits after the prompt."""
    out = None
    for i in range(0, len(ids), tokens):
        out = forward(ids[i:i + tokens], list(range(i, min(i + tokens, len(ids)))), w, c, caches)
    return out


def kv_cache(c, size, zeros=np.zeros):
    """A [2*kv, size, hd] cache per block: keys' heads then values' (models/llama.py:506-514)."""
    return [zeros((2 * c.kv, size, head(c))) for _ in range(c.layers)]


# ---------------------------------------------------------------- seeded synthetic weights

def synthetic(c, seed=0, norm_sigma=0.0, embed_sigma=0.02):
    """Random weights in c's shapes, drawn in a fixed order from default_rng(seed): per block
    qkv_proj, o_proj, then gate_up_proj/down_proj or router/experts.gate_up/experts.down, then embed.
    Linear weights N(0, 0.02) rounded to bf16; norm weights 1 (+ N(0, norm_sigma)); returns
    name -> float32 arrays (bf16 values) including cos / sin tables and embed.T."""
    rng = np.random.default_rng(seed)
    hd, d = head(c), c.dim
    nh = c.heads + 2 * c.kv
    bf = _bfp.bf16_round
    draw = lambda *shape, s=0.02: bf(rng.normal(0, s, shape).astype(np.float32))
    ones = lambda *shape: bf(np.ones(shape, np.float32) + (rng.normal(0, norm_sigma, shape) if norm_sigma else 0))
    w = {}
    for l in range(c.layers):
        pre = f"layers.{l}."
        w[pre + "input_layernorm"] = ones(1, d)
        w[pre + "post_attention_layernorm"] = ones(1, d)
        w[pre + "qkv_proj"] = draw(d, nh * hd)
        w[pre + "o_proj"] = draw(c.heads * hd, d)
        if c.qk_norm:
            qn, kn = ones(1, hd), ones(1, hd)
            w[pre + "qk_norm"] = np.stack([qn] * c.heads + [kn] * c.kv + [np.ones((1, hd), np.float32)] * c.kv)
            w[pre + "qk_on"] = np.array([1.0] * (c.heads + c.kv) + [0.0] * c.kv, np.float32).reshape(nh, 1, 1)
        if c.experts:
            w[pre + "router"] = draw(d, c.experts)
            w[pre + "experts.gate_up"] = draw(c.experts, d, 2 * c.moe)
            w[pre + "experts.down"] = draw(c.experts, c.moe, d)
        else:
            w[pre + "gate_up_proj"] = draw(d, 2 * c.ffn)
            w[pre + "down_proj"] = draw(c.ffn, d)
    w["norm"] = ones(1, d)
    w["embed"] = draw(c.vocab, d, s=embed_sigma)
    w["embed.T"] = np.ascontiguousarray(w["embed"].T)
    w["cos"], w["sin"] = rotary(c, c.places)
    return w
