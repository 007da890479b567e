"""The tensor-parallel split on CPU: two gloo ranks each keep what llama.tp_keep gives them of a block's weights,
compute their partial block in numpy, all-reduce, and must get the one-device result (what the NCCL ranks do on GPUs)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import llama as ollama


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ferrite_b200 import llama
    full = llama.model(dim=64, heads=8, kv=4, layers=1, vocab=256, ffn=96, eps=1e-5, theta=10000.0)
    hd = llama.head(full)
    rng = np.random.default_rng(0)  # every rank draws the same whole matrices
    w = {"qkv_proj": rng.normal(0, 0.1, (64, (8 + 8) * hd)), "o_proj": rng.normal(0, 0.1, (8 * hd, 64)),
         "gate_up_proj": rng.normal(0, 0.1, (64, 192)), "down_proj": rng.normal(0, 0.1, (96, 64)), "embed.T": rng.normal(0, 0.1, (64, 256))}
    x = rng.normal(0, 1, (5, 64))
    mine = {k: np.take(v, llama.tp_keep(k, full, rank, world)[1], llama.tp_keep(k, full, rank, world)[0]) for k, v in w.items()}
    local = llama.tensor_parallel(full, rank, world)
    assert (local.heads, local.kv, local.ffn, local.vocab_shard) == (4, 2, 48, 128)
    # attention's head-wise part: this rank's q heads (their "attention output" here: q itself) through its rows of o_proj
    q_mine = (x @ mine["qkv_proj"])[:, :local.heads * hd]
    partial = q_mine @ mine["o_proj"] + ollama.glu(*np.split(x @ mine["gate_up_proj"], 2, 1)) @ mine["down_proj"]
    total = torch.from_numpy(partial.copy())
    dist.all_reduce(total)
    q_full = (x @ w["qkv_proj"])[:, :8 * hd]
    want = q_full @ w["o_proj"] + ollama.glu(*np.split(x @ w["gate_up_proj"], 2, 1)) @ w["down_proj"]
    ok = np.allclose(total.numpy(), want, rtol=1e-10, atol=1e-10)
    # k and v heads: the ranks' kept columns partition the whole matrix; the vocabulary shards' best picks give the pick
    kept = [torch.zeros(mine["qkv_proj"].shape[1], dtype=torch.int64) for _ in range(world)]
    dist.all_gather(kept, torch.from_numpy(llama.tp_keep("qkv_proj", full, rank, world)[1]))
    ok &= sorted(torch.cat(kept).tolist()) == list(range(w["qkv_proj"].shape[1]))
    logits = x @ mine["embed.T"]
    best = torch.from_numpy(np.stack([logits.max(1), logits.argmax(1) + rank * local.vocab_shard], 1))
    every = [torch.zeros_like(best) for _ in range(world)]
    dist.all_gather(every, best)
    stacked = torch.stack(every)  # [world, tokens, 2]
    pick = stacked[stacked[:, :, 0].argmax(0), torch.arange(5), 1].long().numpy()
    ok &= np.array_equal(pick, (x @ w["embed.T"]).argmax(1))
    if rank == 0:
        result.put(bool(ok))
    dist.destroy_process_group()


def _expert_worker(rank, world, port, result):
    """Expert parallelism as ferrite_b200.llama.experts does it: every rank routes every token, keeps a run of whole
    experts (tp_keep), lists the touched experts among its own and computes a partial sum; the all-reduce gives the
    one-device mixture (oracle.llama.experts)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ferrite_b200 import llama
    E, k, d, F, T = 8, 2, 32, 48, 6
    full = llama.model(dim=d, heads=4, kv=2, layers=1, vocab=256, ffn=0, experts=E, k=k, moe=F, eps=1e-5, theta=10000.0)
    rng = np.random.default_rng(3)
    gate_up, down = rng.normal(0, 0.2, (E, d, 2 * F)), rng.normal(0, 0.2, (E, F, d))
    h = rng.normal(0, 1, (T, d))
    logits = h @ rng.normal(0, 0.5, (d, E))
    values, ids = ollama.topk(logits, k)
    wts = ollama.softmax(values)
    want = ollama.experts(h, {"experts.gate_up": gate_up, "experts.down": down}, ids, wts)
    axis, kept = llama.tp_keep("layers.0.experts.gate_up", full, rank, world)
    assert axis == 0 and llama.tp_keep("layers.0.experts.down", full, rank, world)[1].tolist() == kept.tolist()
    assert llama.tp_keep("layers.0.router", full, rank, world) is None
    mine_gu, mine_down = gate_up[kept], down[kept]
    # what fb_touched(first=...) lists on this rank: its own touched experts numbered from 0, other ranks' picks ignored
    first, mine = rank * len(kept), len(kept)
    ids_here = np.where((ids >= first) & (ids < first + mine), ids - first, mine)
    picks, weights = ollama.touched(ids_here, wts, mine)
    partial = np.zeros((T, d))
    for slot, e in enumerate(np.asarray(picks).reshape(-1)):
        if e < mine:
            x = h @ mine_gu[e]
            partial += (ollama.glu(x[:, :F], x[:, F:]) * np.asarray(weights)[slot].reshape(T, 1)) @ mine_down[e]
    total = torch.from_numpy(partial.copy())
    dist.all_reduce(total)
    ok = np.allclose(total.numpy(), np.asarray(want, dtype=np.float64).reshape(T, d), rtol=1e-9, atol=1e-9)
    every = [torch.zeros(len(kept), dtype=torch.int64) for _ in range(world)]
    dist.all_gather(every, torch.from_numpy(np.asarray(kept, dtype=np.int64)))
    ok &= sorted(torch.cat(every).tolist()) == list(range(E))
    if rank == 0:
        result.put(bool(ok))
    dist.destroy_process_group()


def test_two_ranks_of_experts_reproduce_the_mixture():
    ctx = mp.get_context("spawn")
    result, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_expert_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert result.get(timeout=5) is True


def test_two_ranks_reproduce_one_device():
    ctx = mp.get_context("spawn")
    result, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert result.get(timeout=5) is True


def test_key_heads_shared_by_ranks_when_there_are_fewer_of_them():
    # eight ranks on four key heads: ranks 2j and 2j + 1 both keep key head j (and its values) and share out its query
    # heads; every rank's attention over its own heads, through its rows of o_proj, sums to the whole block's
    from ferrite_b200 import llama
    full = llama.model(dim=64, heads=16, kv=4, layers=1, vocab=1024, ffn=64, eps=1e-5, theta=10000.0)
    hd, world = llama.head(full), 8
    rng = np.random.default_rng(1)
    wqkv, wo, x = rng.normal(0, 0.1, (64, (16 + 8) * hd)), rng.normal(0, 0.1, (16 * hd, 64)), rng.normal(0, 1, (3, 64))

    def heads_out(qkv, H, KV):  # every query head's softmax(q k^T) v over the call's own tokens, side by side
        q, k, v = (ollama.split_heads(qkv[:, a * hd:b * hd], b - a) for a, b in ((0, H), (H, H + KV), (H + KV, H + 2 * KV)))
        k, v = np.repeat(k, H // KV, 0), np.repeat(v, H // KV, 0)
        return ollama.merge_heads(ollama.softmax(q @ k.swapaxes(-1, -2)) @ v)

    want = heads_out(x @ wqkv, 16, 4) @ wo
    total = 0
    for rank in range(world):
        local = llama.tensor_parallel(full, rank, world)
        assert (local.heads, local.kv) == (2, 1)
        cols = llama.tp_keep("qkv_proj", full, rank, world)[1]
        assert cols[2 * hd:3 * hd].tolist() == list(range((16 + rank // 2) * hd, (16 + rank // 2 + 1) * hd))
        rows = llama.tp_keep("o_proj", full, rank, world)[1]
        total = total + heads_out(x @ wqkv[:, cols], 2, 1) @ wo[rows]
    assert np.allclose(total, want, rtol=1e-10, atol=1e-12)


def _dispatch_worker(rank, world, port, result):
    """The all-to-all dispatch of ferrite_b200.llama.experts_dispatched, its layout restated in numpy over two gloo
    ranks: each rank routes its OWN tokens, sends every rank a buffer of tokens x k slots (slot (t, j) real in the
    owner's buffer, "none" elsewhere), runs its experts over what it receives, returns the rows in place, and the sender
    adds its choices' rows by their weights - against the one-device mixture (oracle.llama.moe) on those tokens."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(3)
    d, E, F, k, n = 32, 8, 16, 2, 5
    full = ollama.model(dim=d, experts=E, k=k, moe=F)
    p = {"router": rng.normal(0, 0.5, (d, E)), "experts.gate_up": rng.normal(0, 0.2, (E, d, 2 * F)), "experts.down": rng.normal(0, 0.2, (E, F, d))}
    h = np.random.default_rng(10 + rank).normal(0, 1, (n, d))  # this rank's own tokens
    e = E // world
    vals, ids = ollama.topk(h @ p["router"], k)
    w = ollama.softmax(vals)
    owner, cap = ids // e, n * k
    send = np.zeros((world, cap, d))
    meta = np.full((world, cap), e)
    for t in range(n):
        for j in range(k):
            send[:, t * k + j] = h[t]
            meta[owner[t, j], t * k + j] = ids[t, j] - owner[t, j] * e
    def exchange(a):  # all-to-all by an all-gather (every rank takes its own slice of everyone's buffers)
        every = [torch.zeros_like(torch.from_numpy(a)) for _ in range(world)]
        dist.all_gather(every, torch.from_numpy(a.copy()))
        return np.stack([x.numpy()[rank] for x in every])
    recv, rmeta = exchange(send), exchange(meta)
    back = np.zeros_like(recv)
    for r in range(world):
        for s in range(cap):
            if rmeta[r, s] < e:
                g = recv[r, s] @ p["experts.gate_up"][rank * e + rmeta[r, s]]
                back[r, s] = ollama.glu(g[:F], g[F:]) @ p["experts.down"][rank * e + rmeta[r, s]]
    ret = exchange(back)
    out = np.stack([sum(w[t, j] * ret[owner[t, j], t * k + j] for j in range(k)) for t in range(n)])
    ok = torch.tensor([int(np.allclose(out, ollama.moe(h, p, full), rtol=1e-10, atol=1e-12))])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        result.put(bool(ok.item()))
    dist.destroy_process_group()


def test_two_ranks_dispatch_tokens_to_their_experts():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dispatch_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert result.get(timeout=5)
