"""Tensor parallelism on two, four and eight GPUs: the ranks' sharded decoder (NCCL all-reduce after o_proj and down_proj, sharded
vocabulary pick) must give the single-GPU decoder's tokens and logits - for a dense decoder and for a mixture whose
experts are spread over the ranks (all-reduce after the experts).  With eight ranks the model's four key heads are
each kept by two ranks.  A world larger than the box's GPU count is skipped."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


MODELS = {
    "dense": (dict(dim=512, heads=8, kv=4, layers=2, vocab=1024, ffn=1024, eps=1e-5, theta=10000.0, places=64), "bfp8"),
    "mixture": (dict(dim=512, heads=8, kv=4, layers=2, vocab=1024, ffn=0, experts=8, k=2, moe=256, norm_topk=True, eps=1e-5, theta=10000.0, places=64),
                "experts"),
}


def _worker(rank, world, port, result, kind="dense", peer=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Runtime, Tensor, jit
    rt = Runtime(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=rt.device)
    full = llama.model(**MODELS[kind][0])
    prec = llama.precision(full, MODELS[kind][1])
    c = llama.tensor_parallel(full, rank, world, dist.group.WORLD)
    if peer:  # this library's reduction over NVLink peer memory instead of NCCL's all-reduce
        llama.peer_reduce(rt, c, 4)
    w = llama.random_weights(rt, c, prec, seed=5, full=full, scale=0.05)
    S, part = 4, 32
    on = lambda row: Tensor.of(rt, [row], "int32")
    kv = llama.kv_cache(c, S * part, llama.zeros(rt))
    step = jit(lambda ids, places: llama.next_tokens(llama.forward(ids, places, w, c, kv, S), c))
    ids, picks = [3, 500, 77, 1000], []
    for i in range(5):
        out = step(on(ids), on([i] * S))
        ids = out.numpy().reshape(-1).tolist()
        picks.append(ids)
    if rank == 0:  # the same model on one GPU
        full.vocab_shard = full.vocab
        w1 = llama.random_weights(rt, full, prec, seed=5, scale=0.05)
        kv1 = llama.kv_cache(full, S * part, llama.zeros(rt))
        step1 = jit(lambda ids, places: llama.forward(ids, places, w1, full, kv1, S))
        ids, agree, worst = [3, 500, 77, 1000], 0, 0.0
        for i in range(5):
            logits = step1(on(ids), on([i] * S)).numpy()[0]
            for u in range(S):  # the ranks' pick is the best logit, or one a bf16 rounding apart from it
                worst = max(worst, float(logits[u].max() - logits[u][picks[i][u]]) / float(np.ptp(logits[u])))
            agree += sum(int(logits[u].argmax()) == picks[i][u] for u in range(S))
            ids = picks[i]  # teacher-forced with the ranks' picks
        result.put((agree, worst))
        import time
        time.sleep(1)  # let the queue's feeder thread send before the hard exit
    if peer:
        c.tp.peer.check()
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)  # (no NCCL teardown: the recorded graphs still hold its kernels)


def _ep_worker(rank, world, port, result):
    """A mixture with its experts AND its sequences shared out (llama.expert_parallel): every rank decodes its own two
    sequences, tokens reach their experts by all-to-all, and each rank checks its sequences against the one-GPU decoder."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    from ferrite_b200 import llama
    from ferrite_b200.tensor import Runtime, Tensor, jit
    rt = Runtime(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=rt.device)
    full = llama.model(**MODELS["mixture"][0])
    full.vocab_shard = full.vocab
    prec = llama.precision(full, MODELS["mixture"][1])
    c = llama.expert_parallel(full, rank, world, dist.group.WORLD)
    w = llama.random_weights(rt, c, prec, seed=5, full=full, scale=0.05)
    assert w["layers.0.experts.gate_up"].batch == full.experts // world and w["layers.0.qkv_proj"].cols == (8 + 2 * 4) * 64
    S, part = 2, 32
    on = lambda row: Tensor.of(rt, [row], "int32")
    kv = llama.kv_cache(c, S * part, llama.zeros(rt))
    step = jit(lambda ids, places: llama.forward(ids, places, w, c, kv, S))
    w1 = llama.random_weights(rt, full, prec, seed=5, scale=0.05)  # the same model whole, on this GPU
    kv1 = llama.kv_cache(full, S * part, llama.zeros(rt))
    step1 = jit(lambda ids, places: llama.forward(ids, places, w1, full, kv1, S))
    ids, worst = [3 + 100 * rank, 500 + rank], 0.0
    for i in range(5):  # eager, recorded, replayed; teacher-forced with the whole model's picks
        got, want = step(on(ids), on([i] * S)).numpy()[0], step1(on(ids), on([i] * S)).numpy()[0]
        worst = max(worst, float(np.abs(got - want).max() / np.ptp(want)))
        ids = [int(v) for v in want.argmax(-1)]
    flag = torch.tensor([worst], device=rt.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if rank == 0:
        result.put(float(flag.item()))
        import time
        time.sleep(1)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_experts_and_sequences_shared_out_by_all_to_all(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.kill()
        p.join(10)
    assert not stuck and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=5) < 0.02, "every rank's logits within 2 % of the whole model's span"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kind,peer", [("dense", False), ("mixture", False), ("dense", True), ("mixture", True)])
def test_ranks_decode_like_one_gpu(cuda, kind, peer, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result, kind, peer)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:  # a rank that never came back must not keep its GPU
        p.kill()
        p.join(10)
    assert not stuck and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    agree, worst = result.get(timeout=5)
    assert worst < 0.01 and agree >= 18, (agree, worst)
