"""Decode throughput of the block-float hot path on B200s, one JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama8b|smollm] [--layers L] [--impl reference]
    python bench.py --matmul 32,4096,14336,bfp8,6      (one isolated matmul, a few calls: what the ncu captures run)
    python bench.py --attend 32,32,8,128,2048,6        (the decode attention alone, likewise)

The default workload is the Llama-3.1-8B-shape batched decode (32 sequences, 2048 tokens of context each, bfp8 weights,
bf16 KV cache), tensor-parallel over N GPUs with an NCCL all-reduce after o_proj and down_proj.  A step is one decode
step of all the sequences: embedding gather, 32 blocks (fused RMSNorm + qkv matmul, RoPE + KV write, split-KV attention,
o_proj + residual, RMSNorm + gate_up + SwiGLU, down_proj + residual), final norm, output layer, greedy pick.

    value      tokens/s with the step's inputs resident on the device (the pick of one step feeds the next on the device)
    e2e        the same through the public call with host buffers: ids and places copied in from pinned memory and the
               picked tokens read back, every step
    roofline   the block-float matmul kernel (the dominant kernel): its algorithmic bytes over its measured duration
    matmul_sweep  (1 GPU) the isolated matmul with fused RMSNorm and SwiGLU over M, N and both formats: GB/s and fraction of peak
    cpu_baseline / --impl reference: the numpy restatement of the reference's CPU path on this box's host cores, on a
               bounded sample (one block and the output layer, scaled to the model)
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE.json configs[2]: Llama-3.1-8B shape
    "llama8b": dict(model=dict(dim=4096, heads=32, kv=8, layers=32, vocab=128256, ffn=14336, theta=500000.0, eps=1e-5), mode="bfp8",
                    sequences=32, context=2048, name="llama-3.1-8b-shape bfp8, 32 sequences x 2048 context, bf16 KV"),
    # BASELINE.json configs[0]: SmolLM-135M shape, batch 1 (the reference's own CPU-runnable case)
    # BASELINE.json configs[3]: Mixtral-8x7B shape, attention bfp8, experts bfp4, 64 sequences x 1024 context (one GPU holds it)
    "mixtral": dict(model=dict(dim=4096, heads=32, kv=8, layers=32, vocab=32000, ffn=0, experts=8, k=2, moe=14336, norm_topk=True, theta=1000000.0, eps=1e-5),
                    mode="experts", sequences=64, context=1024, name="mixtral-8x7b-shape, attention bfp8 / experts bfp4, top-2 of 8, 64 sequences x 1024 context, bf16 KV"),
    # BASELINE.json configs[4]: Qwen3-30B-A3B shape, bfp8, 128 sessions with contexts drawn uniformly from 256..8192 (seeded)
    "qwen3moe": dict(model=dict(dim=2048, heads=32, kv=4, head_dim=128, layers=48, vocab=151936, ffn=0, experts=128, k=8, moe=768, norm_topk=True, qk_norm=True,
                                theta=1000000.0, eps=1e-6),
                     mode="bfp8", sequences=128, context=8192, ragged=(256, 8192),
                     name="qwen3-30b-a3b-shape bfp8, top-8 of 128, QK-norm, 128 sessions with contexts U{256..8192}, ragged bf16 KV"),
    "smollm": dict(model=dict(dim=576, heads=9, kv=3, layers=30, vocab=49152, ffn=1536, theta=10000.0, eps=1e-5, tied=True), mode="bfp8",
                   sequences=1, context=32, name="smollm-135m-shape bfp8, batch 1, 32-token prompt, bf16 KV"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="llama8b", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="fewer blocks than the model has (a smoke run; the JSON line says so)")
    ap.add_argument("--impl", default="ferrite_b200", choices=["ferrite_b200", "reference"])
    ap.add_argument("--reduce", default="peer", choices=["peer", "nccl"], help="several GPUs: how the ranks' partial sums are added")
    ap.add_argument("--parallel", default="tp", choices=["tp", "ep"],
                    help="several GPUs: tp = heads / MLP columns / experts sharded, every rank decodes every sequence, all-reduce after o_proj and "
                         "the MLP; ep (mixtures) = experts AND sequences shared out, whole attention on every rank, tokens to their experts by all-to-all")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "bfp8", "bfp4"], help="the KV cache's format (BASELINE.json's configs keep it in bf16)")
    ap.add_argument("--sweep", type=int, default=1, help="0: leave the isolated matmul sweep out of the line (a profiling run)")
    ap.add_argument("--attend", default="", help="T,H,KV,hd,context[,calls]: only the decode attention, e.g. 32,32,8,128,2048,6")
    ap.add_argument("--matmul", default="", help="M,K,N,fmt[,calls]: only that isolated matmul (RMSNorm + SwiGLU fused), e.g. 32,4096,14336,bfp8,6")
    return ap.parse_args()


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class Clocks(threading.Thread):
    """SM clock and throttle reasons sampled through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        import pynvml
        self.nv, self.samples, self.reasons, self.stop = pynvml, [], set(), False
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(index)

    def run(self):
        nv = self.nv
        names = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown", nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
        while not self.stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.reasons |= {n for bit, n in names.items() if mask & bit}
            except Exception:  # a sample that cannot be read is left out
                pass
            time.sleep(0.05)

    def summary(self):
        self.stop = True
        nv = self.nv
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)), "reasons": sorted(self.reasons)}


def linear_bytes(c, sequences, fmt_bytes=1.0625, expert_bytes=None):
    """Algorithmic bytes of one step's block-float matmuls: packed weights once, activations in and out (bf16).  A mixture
    reads the experts some token picked: E (1 - (1 - k/E)^T) of them expected (the reference's cost model, ferrite/cost.py:91)."""
    hd = c.head_dim or c.dim // c.heads
    shapes = [(c.dim, (c.heads + 2 * c.kv) * hd, (c.heads + 2 * c.kv) * hd, fmt_bytes), (c.heads * hd, c.dim, c.dim, fmt_bytes)]
    launches = 2
    if getattr(c, "experts", 0):
        tp = getattr(c, "tp", None) or getattr(c, "ep", None)  # expert parallel: a rank reads its share of the touched experts
        everyone = sequences * (tp.world if getattr(c, "ep", None) else 1)  # (c.ep: the other ranks' sequences pick this rank's experts too)
        touched = c.experts * (1 - (1 - c.k / c.experts) ** max(everyone, 1)) / (tp.world if tp else 1)
        eb = expert_bytes or fmt_bytes
        shapes += [(c.dim, c.experts, c.experts, 2.0), (c.dim, touched * 2 * c.moe, touched * c.moe, eb), (touched * c.moe, c.dim, c.dim, eb)]
        launches += 3
    else:
        shapes += [(c.dim, 2 * c.ffn, c.ffn, fmt_bytes), (c.ffn, c.dim, c.dim, fmt_bytes)]
        launches += 2
    per_layer = sum(k * n * b + 2 * sequences * k + 2 * sequences * out for k, n, out, b in shapes)
    head = c.dim * c.vocab_shard * fmt_bytes + 2 * sequences * c.dim + 4 * sequences * c.vocab_shard
    return c.layers * per_layer + head, launches * c.layers + 1


def step_bytes(c, sequences, context_rows, expert_bytes=None, kv_bytes=2.0):
    """Algorithmic bytes a decode step reads per GPU: weights once, the KV rows each token sees (context_rows: their sum
    over the sequences), its embedding row."""
    hd = c.head_dim or c.dim // c.heads
    weights, _ = linear_bytes(c, sequences, expert_bytes=expert_bytes)
    weights -= c.layers * 0  # (activations are part of linear_bytes; they are negligible)
    kv = context_rows * c.layers * 2 * c.kv * hd * kv_bytes
    return weights + kv + sequences * c.dim * 2


def run_ferrite(args):
    import torch
    import torch.distributed as dist
    from ferrite_b200 import llama, ops
    from ferrite_b200.tensor import Runtime, Tensor, jit

    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run --nproc-per-node {args.gpus}"
    rt = Runtime(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=rt.device)
    wl = WORKLOADS[args.workload]
    full = llama.model(**wl["model"], places=wl["context"] + args.steps + args.warmup + 64)
    if args.layers:
        full.layers = args.layers
    ep = world > 1 and args.parallel == "ep"
    assert not ep or (getattr(full, "experts", 0) and wl["sequences"] % world == 0), "--parallel ep: a mixture, its sequences shared out evenly"
    c = llama.expert_parallel(full, rank, world, dist.group.WORLD) if ep else llama.tensor_parallel(full, rank, world, dist.group.WORLD) if world > 1 else full
    if world == 1:
        c.vocab_shard = full.vocab
    reduction = "none"
    if ep:
        reduction = "none (two all-to-alls a block: tokens to their experts' ranks and back)"
    elif world > 1:
        reduction = "nccl all-reduce + add"
        if args.reduce == "peer":
            why = ""
            try:  # this library's kernel over NVLink peer memory; NCCL's all-reduce if the mapping cannot be set up here
                llama.peer_reduce(rt, c, wl["sequences"])
            except Exception as e:  # noqa: BLE001
                why = type(e).__name__
            ok = torch.tensor([0 if why else 1], device=rt.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # every rank takes the same path
            if int(ok.item()):
                reduction = "fb_peer_reduce_add (own kernel, peer loads over NVLink, residual fused)"
            else:
                c.tp.peer = None
                reduction += f" (peer memory unavailable on some rank{': ' + why if why else ''})"
    prec = llama.precision(full, wl["mode"])
    w = llama.random_weights(rt, c, prec, seed=0, full=full)
    S_all, ctx = wl["sequences"], wl["context"]
    S = S_all // world if ep else S_all  # the sequences this rank decodes
    part = ctx + args.steps + args.warmup + 64
    part += -part % 64
    rng = np.random.default_rng(0)
    # where each sequence stands: all at `context`, or (a serving mix) contexts drawn uniformly, seeded
    ctxs = [int(v) for v in rng.integers(wl["ragged"][0], wl["ragged"][1] + 1, S_all)] if wl.get("ragged") else [ctx] * S_all
    ctxs = ctxs[rank * S:(rank + 1) * S] if ep else ctxs
    moe = bool(getattr(full, "experts", 0))
    expert_bytes = 0.5625 if wl["mode"] == "experts" else None
    hd = llama.head(full)
    caches = []
    gen = torch.Generator(device=rt.device).manual_seed(1 + rank)
    for _ in range(full.layers):  # the prompts' keys and values: N(0, 1), as a prefill would have left them
        t = Tensor(rt, S * part, hd, batch=2 * c.kv)
        t.buf.normal_(0, 1, generator=gen)
        caches.append(t if args.kv == "bf16" else t.cast(args.kv).realize())  # (a block-float cache: rounded as a put rounds)
    kv_bytes = {"bf16": 2.0, "bfp8": 1.0625, "bfp4": 0.5625}[args.kv]
    slots = S if S > 1 else None

    def step_fn(ids, places):
        return llama.next_tokens(llama.forward(ids, places, w, c, caches, slots), c)

    step = jit(step_fn)
    on = lambda row: Tensor.of(rt, [row], "int32")
    ids0 = [int(v) for v in rng.integers(0, full.vocab, S_all)]
    ids0 = ids0[rank * S:(rank + 1) * S] if ep else ids0
    place = 0  # steps taken so far: sequence u stands at ctxs[u] + place
    at = lambda: [v + place for v in ctxs]
    # the first two calls plan and record; they are part of the warm-up
    before = ops.KERNELS[0]
    picks = step(on(ids0), on(at()))
    place += 1
    per_step = None
    for i in range(max(args.warmup, 3) - 1):
        k0 = ops.KERNELS[0]
        picks = step(on(picks.numpy().reshape(-1).tolist()), on(at()))
        if i == 0:
            per_step = ops.KERNELS[0] - k0  # kernels the recorded step holds (counted while it was recorded)
        place += 1
    rt.wait()

    # ---- device-resident loop: the pick feeds the next step on the device, places advance on the device
    ids_t, places_t = on(picks.numpy().reshape(-1).tolist()), on(at())
    one = Tensor.of(rt, [[1] * S], "int32")
    bump = jit(lambda p: p + one)  # (records on its second call)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        places_t = bump(places_t)
    clocks = Clocks(local)
    clocks.start()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step(ids_t, places_t)
        ids_t.buf.copy_(out.buf, non_blocking=True)
        places_t = bump(places_t)
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    place += args.steps + 3

    # ---- end to end: host ids and places in (pinned), picked tokens out, every step
    h_ids = torch.tensor([ids0], dtype=torch.int32).pin_memory()
    h_places = torch.tensor([at()], dtype=torch.int32).pin_memory()
    h_out = torch.empty(1, 1, S, dtype=torch.int32).pin_memory()
    d_ids, d_places = on(ids0), on(at())
    e2e_steps = max(8, args.steps // 2)
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(e2e_steps):
        d_ids.buf.copy_(h_ids.view(1, 1, S), non_blocking=True)
        d_places.buf.copy_(h_places.view(1, 1, S), non_blocking=True)
        out = step(d_ids, d_places)
        h_out.copy_(out.buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_ids.copy_(h_out.view(1, S))  # the next step's input is this step's pick, from the host
        h_places += 1
    e3.record()
    sync_all()
    ms_e2e = e2.elapsed_time(e3)
    clk = clocks.summary()
    if getattr(getattr(c, "tp", None), "peer", None) is not None:
        c.tp.peer.check()

    mm = None
    lin_bytes, lin_launches = linear_bytes(c, S, expert_bytes=expert_bytes)
    lin_ms = 0.0
    # ---- the dominant kernel alone: the step's block-float matmuls, back to back, every weight of the model once
    # (a dense model; a mixture's indexed matmuls depend on the router's picks, so its roofline is the whole step's)
    if not moe:
        x32 = Tensor.of(rt, rng.normal(0, 1, (S, full.dim)).astype(np.float32).tolist())
        f32 = Tensor.of(rt, rng.normal(0, 1, (S, c.ffn)).astype(np.float32).tolist())
        a32 = Tensor.of(rt, rng.normal(0, 1, (S, c.heads * hd)).astype(np.float32).tolist())

        def matmuls():
            for p in w["_blocks"]:
                x32.matmul(p["qkv_proj"]).realize()
                a32.matmul(p["o_proj"]).realize()
                x32.matmul(p["gate_up_proj"]).realize()
                f32.matmul(p["down_proj"]).realize()
            return x32.matmul(w["embed.T"], dtype="fp32").realize()

        mm = jit(lambda: matmuls())
        for _ in range(3):
            mm()
        torch.cuda.synchronize()
        e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        e4.record()
        for _ in range(reps):
            mm()
        e5.record()
        torch.cuda.synchronize()
        lin_ms = e4.elapsed_time(e5) / reps

    # ---- time to first token (one GPU, a dense model): one sequence's prompt of `context` tokens from place 0 in chunks of
    # 128 through the same kernels (the matmuls at 128 rows a pass, the prefill-shaped attention), then the greedy pick
    # (the reference's B3, test/benchmark.py:172-181, times the same call on its side)
    ttft = None
    if world == 1 and not moe:
        prompt = [int(v) for v in rng.integers(0, full.vocab, ctx)]
        one = llama.kv_cache(c, part, llama.zeros(rt))
        tries = []
        for _ in range(2):  # (the first pass also plans and allocates)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            first = llama.next_tokens(llama.prefill(prompt, w, c, one, 128, on), c).numpy()
            tries.append(time.perf_counter() - t0)
        ttft = {"ms": 1e3 * tries[-1], "prompt_tokens": ctx, "chunk": 128, "tokens_per_s": ctx / tries[-1],
                "what": "one sequence's prompt from place 0 to its first token on the host, wall clock, second of two passes"}
        del one

    # max over ranks
    times = torch.tensor([ms, ms_e2e, lin_ms], device=rt.device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e, lin_ms = times.tolist()
    peaks, peak_kind = measured_peaks()
    rows_seen = sum(ctxs) + S * (args.warmup + args.steps // 2)  # KV rows the middle step of the timed run reads
    whole = step_bytes(c, S, rows_seen, expert_bytes, kv_bytes)
    if moe:  # the roofline of a mixture's step as a whole: every kernel of it streams weights or KV rows
        lin_bytes, lin_launches, lin_ms = whole, int(per_step or 1), ms / args.steps
    achieved = lin_bytes / (lin_ms * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": S_all * args.steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl["name"], "layers": full.layers, "parallelism": (f"dp{world} (sequences, whole attention) + ep{world} (experts), all-to-all dispatch and return" if ep else
                                                                             f"tp{world}" + (f" (attention heads) + ep{world} (experts), all-reduce after o_proj and after the experts" if moe and world > 1 else "")), "reduction": reduction, "l2": "inputs larger than L2 (every step streams all weights and KV rows)",
                   "weights": "random N(0, 0.02) quantised on the device", "kv": "N(0, 1) %s standing in for the prompts' prefill" % args.kv},
        "e2e": {"value": S_all * e2e_steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * 4 * S_all, "d2h_bytes_per_step": 4 * S_all, "steps": e2e_steps},
        "gpu_launches": int(per_step or 0) * args.steps,
        "clocks": clk,
        "roofline": {"bound": "hbm", "kernel": ("the whole decode step (indexed block-float matmuls + decode attention), %d tokens" if moe else
                                                "linear_tcgen05_kernel / linear_persistent_kernel (block-float dequant GEMM: a CTA per tile, or persistent with at least a tile per SM; %d tokens)") % S, "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peak_kind,
                     "traffic": None if moe else 1.002 * lin_bytes / lin_launches,
                     "traffic_source": "not captured for the whole step" if moe else "algorithmic bytes x 1.002 (DRAM read+write of the ncu capture in profiles/, 4096x14336 bfp8, 32 tokens)",
                     "launches": lin_launches, "us_per_launch": lin_ms * 1e3 / lin_launches, "bytes_per_launch": lin_bytes / lin_launches},
        "step_roofline": {"algorithmic_bytes_per_gpu": whole, "frac_of_hbm": whole / (ms / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"]},
    }
    if ttft:
        line["ttft"] = ttft
    if rank == 0 and world == 1:
        del w, caches, step, mm
        torch.cuda.empty_cache()
        if args.sweep and not moe:
            line["matmul_sweep"] = matmul_sweep(rt.device, peaks["hbm_gbs"])
        line["cpu_baseline"] = cpu_baseline(args, sample_seconds=20)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:  # leave without tearing NCCL down: the recorded graphs still hold its kernels, and a teardown waits on them
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def one_matmul(spec):
    """--matmul: a few eager calls of one isolated matmul over four weight copies (what an ncu capture of the kernel runs)."""
    import torch
    from ferrite_b200 import ops
    parts = spec.split(",")
    M, K, N, fmt, calls = int(parts[0]), int(parts[1]), int(parts[2]), parts[3], int(parts[4]) if len(parts) > 4 else 6
    device, gen = torch.device("cuda:0"), torch.Generator(device="cuda:0").manual_seed(0)
    g = (1 + 0.1 * torch.randn(K, device=device, generator=gen)).bfloat16()
    ws = [ops.quantize((torch.randn(K, N, device=device, generator=gen) * 0.02).bfloat16(), fmt) for _ in range(4)]
    x = torch.randn(M, K, device=device, generator=gen).bfloat16()
    out = torch.empty(M, N // 2, device=device, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(calls):
        ops.linear(x, ws[i % 4], out=out, norm_w=g, eps=1e-5, epilogue="swiglu")
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"matmul": spec, "calls": calls, "us_per_call_eager": e0.elapsed_time(e1) * 1e3 / calls}))


def one_attention(spec):
    """--attend: a few eager calls of the decode attention alone, every sequence at the same context, each call over its
    own KV cache (four of them, together larger than L2): what an ncu capture of the kernel runs."""
    import torch
    from ferrite_b200 import ops
    parts = [int(v) for v in spec.split(",")]
    T, H, KV, hd, ctx, calls = parts[:5] + [parts[5] if len(parts) > 5 else 6]
    device, gen = torch.device("cuda:0"), torch.Generator(device="cuda:0").manual_seed(0)
    part = ctx + 64 - ctx % 64
    caches = [torch.empty(2 * KV, T * part, hd, device=device, dtype=torch.bfloat16).normal_(0, 1, generator=gen) for _ in range(4)]
    q = torch.randn(T, H * hd, device=device, generator=gen).bfloat16()
    base = torch.arange(T, device=device, dtype=torch.int32) * part
    place = torch.full((T,), ctx - 1, device=device, dtype=torch.int32)
    out = torch.empty(T, H * hd, device=device, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(calls):
        ops.decode_attention(q, caches[i % 4], base, place, H, KV, hd, ctx, out=out)
    e1.record()
    torch.cuda.synchronize()
    kv_bytes = T * ctx * 2 * KV * hd * 2
    print(json.dumps({"attend": spec, "calls": calls, "us_per_call_eager": e0.elapsed_time(e1) * 1e3 / calls, "kv_bytes_per_call": kv_bytes}))


def matmul_sweep(device, peak_gbs, calls=200):
    """BASELINE.json configs[1]: the isolated block-float matmul, RMSNorm prologue and SwiGLU epilogue fused, K = 4096,
    M in {1, 8, 32, 128}, N in {4096, 14336}, bfp8 and bfp4.  `calls` back-to-back calls (one recorded graph) rotate
    through distinct weight buffers that together exceed L2 several times, so every call streams its matrix from HBM.
    Algorithmic bytes per call: the packed matrix, the activations in, the result out, the norm's weight."""
    import torch
    from ferrite_b200 import ops
    K, rows, gen = 4096, [], torch.Generator(device=device).manual_seed(0)
    g = (1 + 0.1 * torch.randn(K, device=device, generator=gen)).bfloat16()
    for fmt, per_value in (("bfp8", 1.0625), ("bfp4", 0.5625)):
        for N in (4096, 14336):
            copies = min(48, -(-(512 << 20) // int(K * N * per_value)))
            ws = [ops.quantize((torch.randn(K, N, device=device, generator=gen) * 0.02).bfloat16(), fmt) for _ in range(copies)]
            for M in (1, 8, 32, 128):
                x = torch.randn(M, K, device=device, generator=gen).bfloat16()
                out = torch.empty(M, N // 2, device=device, dtype=torch.bfloat16)
                for i in range(3):
                    ops.linear(x, ws[i % copies], out=out, norm_w=g, eps=1e-5, epilogue="swiglu")
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for i in range(calls):
                        ops.linear(x, ws[i % copies], out=out, norm_w=g, eps=1e-5, epilogue="swiglu")
                graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / calls
                nbytes = K * N * per_value + 2 * M * K + 2 * M * (N // 2) + 2 * K
                rows.append({"fmt": fmt, "M": M, "N": N, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                             "frac": round(nbytes / us / 1e3 / peak_gbs, 3)})
            del ws
            torch.cuda.empty_cache()
    return {"what": "RMSNorm + [M,4096]x[4096,N] + SwiGLU, %d calls rotating weight copies > L2" % calls, "peak_GB/s": peak_gbs, "rows": rows}


def cpu_sample(args, seconds):
    """One decode step of ONE block plus the output layer of the workload on this box's host cores, timed, and scaled to
    the model's block count.  It runs the reference's OWN numpy code (models/llama.py: around, layer, rms - the numpy
    branch its `fns` picks) when oracle/_ref holds it (oracle/make_ref.py put it there from a checkout; kind
    "reference"), else the restatement under oracle/ (kind "port").  Weights are quantised by the C restatement."""
    from oracle import build as obuild
    from oracle import llama as ollama
    from oracle import make_ref
    ref = make_ref.modules()
    wl = WORKLOADS[args.workload]
    fields = {k: v for k, v in wl["model"].items() if k != "tied"} | dict(places=wl["context"] + 64)
    layers = args.layers or fields["layers"]
    oc = ollama.model(**fields | dict(layers=1))
    c = ref[0].model(**{k: v for k, v in fields.items() if k != "qk_norm"} | dict(layers=1)) if ref else oc
    S, ctx = wl["sequences"], wl["context"]
    rng = np.random.default_rng(0)
    ctxs = [int(v) for v in rng.integers(wl["ragged"][0], wl["ragged"][1] + 1, S)] if wl.get("ragged") else [ctx] * S
    hd, nh = ollama.head(oc), oc.heads + 2 * oc.kv
    fmt = "bfp8" if wl["mode"] == "experts" else wl["mode"]
    q = lambda *shape, f=fmt: obuild.bfp_values(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02), f)
    w = {"layers.0.input_layernorm": np.ones((1, oc.dim), np.float32), "layers.0.post_attention_layernorm": np.ones((1, oc.dim), np.float32),
         "layers.0.qkv_proj": q(oc.dim, nh * hd), "layers.0.o_proj": q(oc.heads * hd, oc.dim), "norm": np.ones((1, oc.dim), np.float32)}
    if getattr(oc, "experts", 0):
        ef = "bfp4" if wl["mode"] == "experts" else fmt
        w["layers.0.router"] = (rng.standard_normal((oc.dim, oc.experts), dtype=np.float32) * np.float32(0.02))
        w["layers.0.experts.gate_up"] = np.stack([q(oc.dim, 2 * oc.moe, f=ef) for _ in range(oc.experts)])
        w["layers.0.experts.down"] = np.stack([q(oc.moe, oc.dim, f=ef) for _ in range(oc.experts)])
        if wl["model"].get("qk_norm"):
            w["layers.0.qk_norm"] = np.ones((nh, 1, hd), np.float32)
            w["layers.0.qk_on"] = np.array([1.0] * (oc.heads + oc.kv) + [0.0] * oc.kv, np.float32).reshape(nh, 1, 1)
    else:
        w["layers.0.gate_up_proj"], w["layers.0.down_proj"] = q(oc.dim, 2 * oc.ffn), q(oc.ffn, oc.dim)
    w["embed"] = (rng.standard_normal((oc.vocab, oc.dim), dtype=np.float32) * np.float32(0.02))
    w["embed.T"] = obuild.bfp_values(np.ascontiguousarray(w["embed"].T), fmt)
    if ref:
        w["cos"], w["sin"], w["turn"] = ref[0].rotary(c, c.places)
    else:
        w["cos"], w["sin"] = ollama.rotary(oc, oc.places)
    part = ctx + 64
    caches = [np.zeros((2 * oc.kv, S * part, hd))]  # np.zeros: float64, as the reference's kv_cache(c, size, np.zeros)
    caches[0][:, :, :] = rng.standard_normal(caches[0].shape)
    ids = [int(v) for v in rng.integers(0, oc.vocab, S)]
    slots = S if S > 1 else None
    threads = blas_threads()
    times, place = [], 0
    start = time.perf_counter()
    while not times or (time.perf_counter() - start < seconds and len(times) < 16):
        t0 = time.perf_counter()
        x = w["embed"][ids]
        places, size = ([v + place for v in ctxs] if slots else [ctx + place]), (S * part if slots else part)
        if ref:
            rows, rotary, mask, _, live = ref[0].around(w, c, places, size, slots)
        else:
            rows, cos, sin, mask, live = ollama.around(w, oc, places, size, slots)
        t_in = time.perf_counter()
        if ref:
            x = ref[0].layer(x, ref[1].block(w, "layers.0."), c, rotary, mask, caches[0], rows, 0, False, live, None, slots)
        else:
            x = ollama.layer(x, ollama.block(w, "layers.0."), oc, cos, sin, mask, caches[0], rows, live, slots)
        t_layer = time.perf_counter()
        logits = (ref[0].rms(x, w["norm"], c) if ref else ollama.rms(x, w["norm"], oc.eps)) @ w["embed.T"]
        picks = logits.argmax(-1)
        t_head = time.perf_counter()
        times.append(((t_in - t0) + (t_head - t_layer), t_layer - t_in))
        place += 1
    rest, layer = np.median([t[0] for t in times]), np.median([t[1] for t in times])
    step_seconds = rest + layers * layer
    return {"value": S / step_seconds, "unit": "tokens/s", "cores": os.cpu_count(), "blas_threads": threads, "kind": "reference" if ref else "port",
            "sample": f"{len(times)} decode steps of 1 of {layers} blocks plus embedding and output layer, "
                      + ("the reference's own models/llama.py numpy branch" if ref else "the numpy restatement of the reference's CPU path")
                      + " (float32 weights, float64 KV cache as the reference keeps it); block time x " + f"{layers} + the rest",
            "seconds_per_step_scaled": step_seconds}


def blas_threads():
    """The threads numpy's BLAS uses (what the CPU legs' matmuls run on), pinned to the host's cores where a launcher
    set it to one (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers)."""
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        want = os.cpu_count() or 1
        threadpool_limits(want)
        return max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:  # noqa: BLE001  (threadpoolctl missing: numpy's default)
        return None


def cpu_baseline(args, sample_seconds):
    return cpu_sample(args, sample_seconds)


def run_reference(args):
    """The reference arm: the reference's CPU path (its numpy branch, restated under oracle/) on this box's host cores."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    wl = WORKLOADS[args.workload]
    base = cpu_sample(args, seconds=min(120, 4 * max(args.steps, 1)))
    S = wl["sequences"]
    line = {"impl": "reference", "metric": "decode tokens/s", "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * S / base["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "layers": args.layers or wl["model"]["layers"], "parallelism": "host cores"},
            "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.matmul:
        one_matmul(a.matmul)
    elif a.attend:
        one_attention(a.attend)
    else:
        run_reference(a) if a.impl == "reference" else run_ferrite(a)
