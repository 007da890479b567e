"""A Llama-family decoder on ferrite_b200 Tensors: the layer calls of the reference's models/llama.py (forward, layer,
attention, mlp, glu, moe, rms, around, kv_cache, precision, weight_format, upload) with the same names, argument meaning
and weight naming, written for the CUDA backend.

The expressions are the reference's (RMSNorm as x * rsqrt(mean(x*x) + eps) * w, SwiGLU as silu(gate) * up, residual adds);
the planner in tensor.py fuses them into the block-float matmuls.  Two steps the reference spells as several ops are one
kernel each here, because their kernels are: RoPE with the KV-cache write (Tensor.rope_put) and attention over the cache
rows a token's place reaches (Tensor.attend_cache); `around` therefore passes places instead of materialised masks, as
the reference does on the chip (models/llama.py:450-452)."""
import math
from types import SimpleNamespace

import numpy as np
import torch

from . import ops
from .tensor import BFP, Tensor, jit  # noqa: F401  (jit re-exported: `from ferrite_b200.llama import jit`)

# a config's fields past a plain Llama's, as a plain Llama has them (models/llama.py:541-543)
DEFAULTS = dict(head_dim=None, rope=None, sliding=None, k=0, experts=0, moe=0, norm_topk=True, tied=False, precision=None, places=4096,
                ffn=None, vocab=None, qk_norm=False, tp=None)


def model(**c):
    return SimpleNamespace(**DEFAULTS | c)


def head(c):
    return c.head_dim or c.dim // c.heads


def precision(c, mode="bf16", kv=None):
    """{(op, block): (format, phases)} (models/llama.py:54-76); the phases are kept for the signature and ignored (the
    products are exact here).  kv: the KV cache's format, under ("kv", None): bf16 unless said, bfp8 for the reference's
    fast modes ("tt", "experts")."""
    four = {"bfp4": ("gate_up",), "tt": ("gate_up",), "experts": ("gate_up", "down")}.get(mode, ())
    fmt = lambda op: mode if mode in ("bf16", "bfp8") else ("bfp4" if op in four else "bfp8")
    p = {(op, l): (fmt(op), 4) for l in range(c.layers) for op in ("qkv", "o", "gate_up", "down")}
    p["head", None] = (fmt("head"), 4)
    p["kv", None] = (kv or ("bfp8" if mode in ("tt", "experts") else "bf16"), None)
    return p


def precision_of(c, op, block=None):
    """(format, phases) of op in block under c.precision, None for either unless said (models/llama.py:78)."""
    return (getattr(c, "precision", None) or {}).get((op, block), (None, None))


def cache_format(c):
    """The KV cache's format under c.precision (models/llama.py:80)."""
    return precision_of(c, "kv")[0] or "bf16"


def weight_format(name, prec):
    """A weight's format on the device (models/llama.py:615-623): matmul B operands per `prec`, the rest bf16."""
    if not prec:
        return "bf16"
    if name == "embed.T":
        return prec.get(("head", None), ("bf16",))[0]
    if name.startswith("layers.") and name.endswith(("_proj", "experts.gate_up", "experts.down")):
        op = name.split(".")[-1].removesuffix("_proj")
        return prec.get((op, int(name.split(".")[1])), ("bf16",))[0]
    return "bf16"


def upload(rt, weights, prec=None):
    """name -> Tensor from name -> numpy arrays of bf16 values, each cast on the device to its format
    (models/llama.py:628-640).  qk_norm / qk_on arrive as the reference stacks them ([heads, 1, hd])."""
    t = {}
    for name, w in weights.items():
        f = weight_format(name, prec)
        if callable(getattr(w, "device", None)):  # a checkpoint's Weight (ferrite_b200/checkpoint.py): made on the device, piece by piece
            x = w.device(rt)
            t[name] = x.cast(f).realize() if f != "bf16" else x
            continue
        a = np.asarray(w, np.float32)
        a = a.reshape((1,) * (3 - a.ndim) + a.shape) if a.ndim <= 3 else a
        x = Tensor.of(rt, a)
        f = weight_format(name, prec)
        t[name] = x.cast(f).realize() if f != "bf16" else x
    return t


def rms(x, w, c):
    """RMSNorm scaled by w (models/llama.py:82-85)."""
    n = x * ((x * x).mean(2) + c.eps).rsqrt()
    return n * w


def glu(gate, up):
    """SwiGLU's silu(gate) * up (models/llama.py:271-275)."""
    return gate.silu() * up


def mlp(h, p, pre=""):
    """silu(h @ gate) * (h @ up), then down; gate and up side by side in gate_up_proj (models/llama.py:266-269)."""
    m = p[pre + "down_proj"].rows
    gate_up = h.matmul(p[pre + "gate_up_proj"])
    return glu(gate_up[:, :m], gate_up[:, m:]).matmul(p[pre + "down_proj"])


def attention(h, p, c, rotary, seen, cache, rows, slots=None):
    """A block's attention over its cache (models/llama.py:111-146).  rotary: (cos, sin) tables and the tokens' places;
    seen: (first cache row of each token's sequence, its last visible key, keys a sequence can hold, window)."""
    cos, sin, places = rotary
    base, last, length, window = seen
    qkv = h.matmul(p["qkv_proj"])
    q = qkv.rope_put(cos, sin, places, rows, cache, c.heads, c.kv, p.get("qk_norm"), c.eps)
    # (a prompt's chunk - several tokens of one sequence - shares its key rows between the tokens of a query head)
    o = q.attend_cache(cache, base, last, c.kv, length, window, chunk=slots is None and q.rows > 1)
    return o.matmul(p["o_proj"])


def moe(h, p, c, live=None):
    """A mixture of experts in the MLP's place (models/llama.py:277-292): router logits, the k best experts and the
    softmax of their logits on the device, then every touched expert's SwiGLU for the step's tokens, weighted and summed
    (the reference's decode form, chip_experts, models/llama.py:302-329)."""
    logits = h.matmul(p["router"], dtype="fp32")  # (fp32: the picks are compared exactly as stored, tensor.py topk)
    if c.norm_topk:
        values, ids = logits.topk(c.k)
        w = values.softmax()
    else:
        w, ids = logits.softmax().topk(c.k)
    return experts(h, p, ids, w if live is None else w * live, c)


def experts(h, p, ids, w, c=None):
    """Expert parallel (c.tp): every rank routes every token (the router is replicated) and holds a run of the experts;
    it lists and runs the touched experts it holds, so its result is a partial sum, reduced over the ranks like a
    row-sharded down_proj's (`added`)."""
    if getattr(c, "ep", None):
        return experts_dispatched(h, p, ids, w, c)
    gate_up, down = p["experts.gate_up"], p["experts.down"]
    m, e = down.rows, gate_up.batch
    tp = getattr(c, "tp", None)
    first, n, k = tp.rank * e if tp else 0, ids.rows, ids.cols
    if n <= 128:  # a decode step: every touched expert an entry, all the tokens its rows (models/llama.py:317-324)
        picks, weights = ids.touched(e, w.bfloat16().realize(), first=first)
        x = h.matmul(gate_up, index=picks)
        g = glu(x[:, :, :m], x[:, :, m:])
        return (g * weights).matmul(down, index=picks).sum(0)
    # a prompt: each expert's tokens grouped into whole tiles of 32, a batch entry a tile, each token's k outputs gathered
    # back, weighted and summed (models/llama.py:318-320, 325-329).  A rank that holds some of the experts groups only the
    # choices among its own; the others' weigh 0 here and are added by the ranks that hold them.
    w = w.bfloat16().realize()
    if tp:
        mine = ((ids >= first) * (ids < first + e)).realize()
        ids, w = ((ids - first) * mine + (1 - mine) * e).realize(), (w * mine.bfloat16()).realize()
    order, picks, places = ids.group(e)
    x = h.realize().gather(order).split(picks.rows, 1)
    x = x.matmul(gate_up, index=picks).realize()
    y = glu(x[:, :, :m], x[:, :, m:]).matmul(down, index=picks).realize().reshape(order.cols, down.cols)
    run = places.cols // k
    terms = [y.gather(places[:, :, j * run:j * run + n]) * w[:, :, j:j + 1] for j in range(k)]
    out = terms[0]
    for term in terms[1:]:
        out = out + term
    return out


def experts_dispatched(h, p, ids, w, c):
    """Expert parallel with the TOKENS shared out too (c.ep, from expert_parallel): every rank decodes its own sequences
    with the whole attention, holds a run of whole experts, and a token's row travels to the ranks that hold its chosen
    experts and its results come back: two all-to-alls over NVLink a block, no all-reduce.  Shapes are fixed, so the step
    records as a CUDA graph: a rank sends every peer one buffer of tokens x k slots, slot (t, j) filled in the buffer of
    the rank that owns token t's choice j and marked "none" in the others; a receiver groups the slots it was sent by
    expert into whole tiles (Tensor.group), runs its experts' SwiGLUs over them, and returns every slot's row in place;
    the sender picks each choice's row out of its owner's buffer and adds them up by their weights.  The reference
    drives one chip and has no counterpart (ferrite/runtime.py:304-311); the arithmetic is numpy_experts'
    (models/llama.py:294-300)."""
    import torch.distributed as dist
    ep, rt = c.ep, h.rt
    gate_up, down = p["experts.gate_up"], p["experts.down"]
    m, e, R = down.rows, gate_up.batch, ep.world
    n, k, d = ids.rows, ids.cols, h.cols
    cap = n * k
    key = ("dispatch", n, k, R)
    if key not in rt.numbers:  # constants of the step's shape: each slot's token, each slot's number, the ranks
        rt.numbers[key] = (Tensor.of(rt, [[t for t in range(n) for _ in range(k)] * R], "int32"),
                           Tensor.of(rt, [[t * k + j for j in range(k)] for t in range(n)], "int32"),
                           Tensor.of(rt, [[[r]] for r in range(R)], "int32"))
    token_of_slot, slot_of, ranks = rt.numbers[key]
    h, ids, w = h.realize(), ids.realize(), w.bfloat16().realize()
    owner = ids >= e  # the rank that holds each choice: how many ranks' runs of experts lie at or below it
    for r in range(2, R):
        owner = owner + (ids >= r * e)
    owner = owner.realize() if R > 1 else (ids * 0).realize()
    here = owner.eq(ranks)  # [R, n, k]: 1 in the buffer of the owner
    meta = ((ids - owner * e) * here + (1 - here) * e).realize()  # the expert's number on its owner, "none" (e) elsewhere
    send = h.gather(token_of_slot)  # [R * cap, d]: every buffer holds every slot's token (only the owner's copy is used)
    recv, rmeta = Tensor(rt, R * cap, d), Tensor(rt, R * cap, 1, dtype="int32")
    dist.all_to_all_single(recv.buf.view(R * cap, d), send.buf.view(R * cap, d), group=ep.group)
    dist.all_to_all_single(rmeta.buf.view(R * cap), meta.buf.view(R * cap), group=ep.group)
    rt.launched("all-to-all dispatch")
    order, picks, places = rmeta.group(e)
    x = recv.gather(order).split(picks.rows, 1)
    x = x.matmul(gate_up, index=picks).realize()
    y = glu(x[:, :, :m], x[:, :, m:]).matmul(down, index=picks).realize().reshape(order.cols, d)
    back, ret = y.gather(places[:, :, :R * cap]), Tensor(rt, R * cap, d)
    dist.all_to_all_single(ret.buf.view(R * cap, d), back.buf.view(R * cap, d), group=ep.group)
    rt.launched("all-to-all return")
    mine = ret.gather((owner * cap + slot_of).realize().reshape(1, 1, cap)).reshape(n, k, d)  # each choice's row, from its owner's buffer
    return (mine * w.reshape(n, k, 1)).sum(1).reshape(1, n, d)


def layer(x, p, c, rotary, seen, cache, rows, live=None, slots=None):
    """One block: attention then a SwiGLU MLP (or a mixture of experts), each after an RMSNorm and added back
    (models/llama.py:95-109).  Tensor-parallel (c.tp): every rank holds its heads' and its MLP columns' share of the
    weights, so o_proj and down_proj give partial sums: an all-reduce over NVLink after each, the residual added once."""
    x = added(x, attention(rms(x, p["input_layernorm"], c), p, c, rotary, seen, cache, rows, slots), c)
    h = rms(x, p["post_attention_layernorm"], c)
    return added(x, moe(h, p, c, live) if "router" in p else mlp(h, p), c)


def added(x, y, c):
    """x + y; with tensor parallelism y is this rank's partial sum: rank 0 adds x, then the ranks' results are summed."""
    tp = getattr(c, "tp", None)
    if not tp:
        return x + y
    peer = getattr(tp, "peer", None)
    if peer is not None and x.batch == 1 and x.dtype == "bf16":
        # this library's kernel over NVLink peer memory: the partial is computed straight into memory every rank maps,
        # then one kernel per rank adds all the partials and the residual (ferrite_b200/peer.py)
        xr = x.realize()
        xr = xr if xr.buf.is_contiguous() else (xr + 0).realize()
        stage = Tensor(x.rt, x.rows, x.cols, buf=peer.stage(x.rows, x.cols))
        y.realize(into=stage)
        out = Tensor(x.rt, x.rows, x.cols)
        peer.reduce_add(x.rows * x.cols, xr.buf, out.buf)
        return out
    import torch.distributed as dist
    out = (x + y if tp.rank == 0 else y).realize()
    if not out.buf.is_contiguous() or out.owner is not None:
        out = (out + 0).realize()
    dist.all_reduce(out.buf, group=tp.group)
    return out


def tensor_parallel(c, rank, world, group=None):
    """c as rank `rank` of `world` holds it: its share of the query and key heads, of the MLP's columns and of the
    vocabulary (models too large or too slow for one GPU; the reference has no counterpart: one chip, ferrite/runtime.py:304-311)."""
    assert c.heads % world == 0 and (c.ffn or 0) % world == 0 and c.vocab % (16 * world) == 0, "shards of whole heads and runs"
    # fewer key heads than ranks: each key head (and its values) is kept by world / kv ranks, which share out its query heads
    assert c.kv % world == 0 or (world % c.kv == 0 and (c.heads // c.kv) % (world // c.kv) == 0), "whole key heads, or whole shares of one key head's queries"
    assert (getattr(c, "experts", 0) or 0) % world == 0, "every rank holds the same number of whole experts"
    local = SimpleNamespace(**vars(c))
    local.head_dim, local.heads, local.kv, local.dim = head(c), c.heads // world, max(c.kv // world, 1), c.dim
    local.ffn, local.vocab_shard = (c.ffn or 0) // world, c.vocab // world
    local.tp = SimpleNamespace(rank=rank, world=world, group=group, peer=None)
    return local


def expert_parallel(c, rank, world, group=None):
    """c as rank `rank` of `world` holds it when a mixture's experts AND its sequences are shared out: the whole attention
    and output layer on every rank (each decodes its own sequences), a run of whole experts each, tokens travelling to
    their experts by all-to-all (experts_dispatched)."""
    assert (getattr(c, "experts", 0) or 0) % world == 0 and c.experts, "a mixture, every rank holding the same number of whole experts"
    local = SimpleNamespace(**vars(c))
    local.ep = SimpleNamespace(rank=rank, world=world, group=group)
    local.vocab_shard = c.vocab
    return local


def peer_reduce(rt, c, tokens):
    """Give c (from tensor_parallel) this library's NVLink reduction for its blocks' partial sums instead of NCCL's
    all-reduce: 2 sites a block, each `tokens` rows of the model's width.  Collective over c.tp.group."""
    from .peer import PeerReduce
    peer = PeerReduce(rt, c.tp.group, tokens * c.dim, 2 * c.layers)
    peer.selftest()
    c.tp.peer = peer
    return c


def tp_keep(name, full, rank, world):
    """What rank `rank` of `world` keeps of the weight called `name`: (axis, indices) into the whole matrix, or None for
    a weight every rank holds whole.  qkv_proj: its heads' columns of q, of k and of v; gate_up_proj: its columns of the
    gate half and of the up half; o_proj and down_proj: the matching rows; embed.T: its run of the vocabulary; a
    mixture's experts: its run of whole experts (the router stays whole on every rank)."""
    hd, H, KV = head(full), full.heads, full.kv
    run = lambda first, size: np.arange(first + rank * (size // world), first + (rank + 1) * (size // world))
    op = name.split(".")[-1]
    if op == "qkv_proj":
        if KV % world:  # fewer key heads than ranks: the one key head this rank's query heads belong to, and its values
            mine = rank * KV // world
            one = lambda first: np.arange(first + mine * hd, first + (mine + 1) * hd)
            return 1, np.concatenate([run(0, H * hd), one(H * hd), one((H + KV) * hd)])
        return 1, np.concatenate([run(0, H * hd), run(H * hd, KV * hd), run((H + KV) * hd, KV * hd)])
    if op == "o_proj":
        return 0, run(0, H * hd)
    if op == "gate_up_proj":
        return 1, np.concatenate([run(0, full.ffn), run(full.ffn, full.ffn)])
    if op == "down_proj":
        return 0, run(0, full.ffn)
    if name == "embed.T":
        return 1, run(0, full.vocab)
    if name.endswith(("experts.gate_up", "experts.down")):
        return 0, run(0, full.experts)
    return None


def next_tokens(out, c):
    """The greedy pick of each row of logits, int32 [1, 1, rows], on the device.  Tensor-parallel: `out` is this rank's
    shard of the vocabulary; each rank picks its best and the ranks' bests are compared (8 bytes a token a rank)."""
    tp = getattr(c, "tp", None)
    if not tp:
        return out.greedy()
    import torch.distributed as dist
    rt, n = out.rt, out.rows
    best = Tensor(rt, 1, n, dtype="fp32")
    ids = (out.greedy(best) + tp.rank * c.vocab_shard).realize()
    all_best, all_ids = Tensor(rt, tp.world, n, dtype="fp32"), Tensor(rt, tp.world, n, dtype="int32")
    dist.all_gather_into_tensor(all_best.buf, best.buf, group=tp.group)
    dist.all_gather_into_tensor(all_ids.buf, ids.buf, group=tp.group)
    _, pick = (all_best.T + 0).realize().topk(1, labels=(all_ids.T + 0).realize())  # the lowest rank (lowest column) among equals
    return pick.reshape(1, 1, n)


def firsts(rt, n, slots, part, cache={}):
    """n tokens' sequences' first rows, n / slots tokens each in turn (models/llama.py:454-457); made once."""
    key = (id(rt), n, slots, part)
    if key not in cache:
        cache[key] = Tensor.of(rt, [[i // (n // slots) * part for i in range(n)]], "int32")
    return cache[key]


def around(w, c, places, size, slots=None, length=None):
    """For tokens at places: their caches' rows, each one's sequence's first row and last visible key, and which tokens
    are live (models/llama.py:429-452).  With slots a free slot's token sits on its part's last row: it is not live and
    sees only its part's first key."""
    n = places.cols
    if not slots:
        zero = firsts(places.rt, n, 1, 0)
        return places, (zero, places, length or size, getattr(c, "sliding", None) or 0), None
    part = size // slots
    base = firsts(places.rt, n, slots, part)
    rows = (places + base).realize()
    at = places.reshape(1, n, 1)
    live = (at < part - 1).bfloat16().realize()
    last = (places * (places < part - 1)).realize()
    return rows, (base, last, length or part, getattr(c, "sliding", None) or 0), live


def block(w, pre):
    return {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}


def forward(ids, places, w, c, caches, slots=None, every=False, length=None):
    """The logits for the token after ids, the tokens at places (models/llama.py:459-480): ids and places int32 row
    tensors; caches each block's keys' heads then its values'; slots: several sequences decoding together, their caches
    side by side, the logits every token's."""
    x = w["embed"].gather(ids)
    if getattr(getattr(c, "tp", None), "peer", None) is not None:
        c.tp.peer.new_step()
    size = caches[0].rows
    rows, seen, live = around(w, c, places, size, slots, length)
    rotary = (w["cos"], w["sin"], places)
    blocks = w.get("_blocks") or [block(w, f"layers.{l}.") for l in range(c.layers)]
    for l in range(c.layers):
        x = layer(x, blocks[l], c, rotary, seen, caches[l], rows, live, slots)
    h = rms(x, w["norm"], c)
    if not (slots or every):
        h = h.realize()[:, x.rows - 1:, :]
    return h.matmul(w["embed.T"], dtype="fp32")


def prefill(ids, w, c, caches, tokens, on):
    """A prompt from place 0 in chunks of `tokens` (models/llama.py:498-504): a chunk's keys and values are in the caches
    before the next chunk attends, so the scores are a chunk's rows by the places so far, never the prompt squared.
    on: makes the int32 row tensor forward takes from a list.  Returns the logits for the token after the prompt."""
    out = None
    for first in range(0, len(ids), tokens):
        chunk = list(ids[first:first + tokens])
        out = forward(on(chunk), on(list(range(first, first + len(chunk)))), w, c, caches)
    return out


def kv_cache(c, size, zeros, slots=1):
    """Each block's keys' heads then its values', a row for each of size places (models/llama.py:506-514)."""
    return [zeros((2 * c.kv, size, head(c))) for _ in range(c.layers)]


def slot(c, caches, u, slots):
    """Caches made for several sequences (slots) as sequence u's alone, in place: its part of each block's cache
    (models/llama.py:520-526).  bf16 caches (a view); a block-float cache's sequences are addressed by their first rows
    (forward's slots) instead."""
    assert all(kv.dtype not in BFP for kv in caches), "a view of a block-float cache's rows: run the sequences together (slots) instead"
    return [kv[:, u * kv.rows // slots:(u + 1) * kv.rows // slots, :] for kv in caches]


def zeros(rt, dtype="bf16"):
    """zeros of a shape on the device, for kv_cache (models/llama.py:656-658)."""
    def make(shape, d=None):
        t = Tensor(rt, shape[1], shape[2], batch=shape[0], dtype=dtype)
        (t.packed.data if dtype in BFP else t.buf).zero_()  # (a block float of zero bytes is zeros)
        return t
    return make


def logits(out):
    """A row of logits as a numpy vector (models/llama.py:655)."""
    return out.numpy()[0, 0]


def frequencies(c):
    hd = head(c)
    inv = 1 / c.theta ** (np.arange(0, hd, 2, dtype=np.float32) / hd)
    r = c.rope
    if r and r.get("rope_type") == "llama3":  # Llama 3's scaling of the long wavelengths (models/llama.py:340-345)
        old, wavelen = r["original_max_position_embeddings"], 2 * math.pi / inv
        scaled = np.where(wavelen > old / r["low_freq_factor"], inv / r["factor"], inv)
        smooth = (old / wavelen - r["low_freq_factor"]) / (r["high_freq_factor"] - r["low_freq_factor"])
        between = (wavelen >= old / r["high_freq_factor"]) & (wavelen <= old / r["low_freq_factor"])
        inv = np.where(between, (1 - smooth) * scaled / r["factor"] + smooth * scaled, scaled).astype(np.float32)
    return inv


def rotary(c, n, wide=False):
    """cos and sin for places 0..n-1 as float32 arrays of bf16 values: angles in fp32, tables rounded to bf16
    (models/llama.py:351-368).  One head's table ([n, hd]; the kernel leaves v's heads unturned), or with wide=True
    the reference's (one per q, k and v head side by side, v's 1 and 0)."""
    hd = head(c)
    angles = np.arange(n, dtype=np.float32)[:, None] * frequencies(c)[None]
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).bfloat16().float().numpy()
    cos, sin = bf(np.concatenate([np.cos(angles)] * 2, 1)), bf(np.concatenate([np.sin(angles)] * 2, 1))
    if not wide:
        return cos, sin
    still = lambda v: np.full((n, hd), v, np.float32)
    return (np.concatenate([cos] * (c.heads + c.kv) + [still(1)] * c.kv, 1), np.concatenate([sin] * (c.heads + c.kv) + [still(0)] * c.kv, 1))


def random_weights(rt, c, prec=None, seed=0, scale=0.02, full=None):
    """Random weights in c's shapes made on the device (for models too large to draw on the host): linear weights
    N(0, scale) rounded to bf16 then cast to their formats, norm weights 1, RoPE tables for c.places places.
    c from tensor_parallel (full: the whole model's config): every rank draws the whole matrices from the same seed and
    keeps its columns or rows, so the ranks together hold exactly the one-GPU model."""
    gen = torch.Generator(device=rt.device).manual_seed(seed)
    full = full or c
    tp = getattr(c, "tp", None) or getattr(c, "ep", None)
    only_experts = getattr(c, "tp", None) is None  # (c.ep: the attention and the output layer are whole on every rank)
    r, n = (tp.rank, tp.world) if tp else (0, 1)
    hd, d = head(full), full.dim
    H, KV = full.heads, full.kv

    def keep(name, x, pick=None):
        if pick is not None:
            x = pick(x).contiguous()
        shape3 = (1,) * (3 - x.dim()) + tuple(x.shape)
        t = Tensor(rt, shape3[1], shape3[2], batch=shape3[0], buf=x.view(shape3))
        f = weight_format(name, prec)
        return t.cast(f).realize() if f != "bf16" else t

    def draw(*shape):
        return torch.empty(*shape, dtype=torch.float32, device=rt.device).normal_(0, scale, generator=gen).bfloat16()

    def mine(name):
        kept = tp_keep(name, full, r, n) if tp and (not only_experts or name.endswith(("experts.gate_up", "experts.down"))) else None
        if kept is None:
            return None
        axis, idx = kept
        index = torch.from_numpy(idx).to(rt.device)
        return lambda x: x.index_select(axis, index)

    ones = lambda m: Tensor.of(rt, np.ones((1, m), np.float32))
    w = {}
    for l in range(full.layers):
        pre = f"layers.{l}."
        w[pre + "input_layernorm"], w[pre + "post_attention_layernorm"] = ones(d), ones(d)
        w[pre + "qkv_proj"] = keep(pre + "qkv_proj", draw(d, (H + 2 * KV) * hd), mine(pre + "qkv_proj"))
        w[pre + "o_proj"] = keep(pre + "o_proj", draw(H * hd, d), mine(pre + "o_proj"))
        if full.qk_norm:
            w[pre + "qk_norm"] = Tensor.of(rt, np.ones((c.heads + c.kv, 1, hd), np.float32))
        if full.experts:
            w[pre + "router"] = keep(pre + "router", draw(d, full.experts))
            w[pre + "experts.gate_up"] = keep(pre + "experts.gate_up", draw(full.experts, d, 2 * full.moe), mine(pre + "experts.gate_up"))
            w[pre + "experts.down"] = keep(pre + "experts.down", draw(full.experts, full.moe, d), mine(pre + "experts.down"))
        else:
            w[pre + "gate_up_proj"] = keep(pre + "gate_up_proj", draw(d, 2 * full.ffn), mine(pre + "gate_up_proj"))
            w[pre + "down_proj"] = keep(pre + "down_proj", draw(full.ffn, d), mine(pre + "down_proj"))
    w["norm"] = ones(d)
    embed = draw(full.vocab, d)
    w["embed"] = Tensor(rt, full.vocab, d, buf=embed.view(1, full.vocab, d))
    w["embed.T"] = keep("embed.T", embed.t(), mine("embed.T") or (lambda x: x))
    cos, sin = rotary(full, full.places)
    w["cos"], w["sin"] = Tensor.of(rt, cos), Tensor.of(rt, sin)
    w["_blocks"] = [block(w, f"layers.{l}.") for l in range(full.layers)]
    return w
