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
