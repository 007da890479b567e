"""bench.py's byte accounting and CPU sample on CPU (no GPU): the algorithmic bytes behind roofline and step_roofline."""
import types

import numpy as np

import bench


def _cfg(**kw):
    base = dict(dim=4096, heads=32, kv=8, head_dim=0, layers=32, vocab_shard=128256, ffn=14336, experts=0, k=0, moe=0)
    return types.SimpleNamespace(**(base | kw))


def test_dense_step_bytes_match_the_hand_count():
    c = _cfg()
    weights, launches = bench.linear_bytes(c, 0)
    values = 32 * (4096 * 6144 + 4096 * 4096 + 4096 * 28672 + 14336 * 4096) + 4096 * 128256
    assert launches == 4 * 32 + 1 and abs(weights - values * 1.0625) < 1e-6 * weights
    rows = 32 * 2048
    kv = rows * 32 * 2 * 8 * 128 * 2
    assert abs(bench.step_bytes(c, 32, rows) - (bench.linear_bytes(c, 32)[0] + kv + 32 * 4096 * 2)) < 1


def test_mixture_reads_only_the_touched_experts():
    c = _cfg(ffn=0, experts=8, k=2, moe=14336, vocab_shard=32000)
    one, _ = bench.linear_bytes(c, 1, expert_bytes=0.5625)
    many, _ = bench.linear_bytes(c, 64, expert_bytes=0.5625)
    expert = 3 * 4096 * 14336 * 0.5625
    assert one < 32 * 2.1 * expert + 3e9 and many > 32 * 7.9 * expert  # 2 of 8 experts for one token, all 8 for 64
    tp = _cfg(ffn=0, experts=8, k=2, moe=14336, vocab_shard=32000, tp=types.SimpleNamespace(world=2))
    assert bench.linear_bytes(tp, 64, expert_bytes=0.5625)[0] < many


def test_cpu_sample_runs_a_mixture_block():
    bench.WORKLOADS["_tiny_moe"] = dict(model=dict(dim=128, heads=4, kv=2, head_dim=32, layers=2, vocab=256, ffn=0, experts=4, k=2, moe=64, norm_topk=True,
                                                     qk_norm=True, theta=1e6, eps=1e-6), mode="experts", sequences=3, context=24, ragged=(8, 24), name="tiny")
    try:
        out = bench.cpu_sample(types.SimpleNamespace(workload="_tiny_moe", layers=0, steps=2, warmup=1), 1)
    finally:
        del bench.WORKLOADS["_tiny_moe"]
    assert out["value"] > 0 and out["kind"] in ("port", "reference") and np.isfinite(out["seconds_per_step_scaled"])
