"""fb_linear: block-float weight matmul with fused RMSNorm prologue and SwiGLU / residual epilogue against
the numpy oracle (the reference's numpy branch: exact products, models/llama.py:33, 82-85, 266-275)."""
import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor, to_numpy
from ferrite_b200 import ops
from oracle import bfp, llama

pytestmark = pytest.mark.gpu


def case(rng, M, K, N, fmt, cuda, sigma=0.02):
    x = bfp.bf16_round(rng.normal(0, 1, (M, K)).astype(np.float32))
    w = bfp.bf16_round(rng.normal(0, sigma, (K, N)).astype(np.float32))
    packed = ops.quantize(to_bf16_tensor(w, cuda), fmt)
    return x, bfp.bfp(w, fmt), to_bf16_tensor(x, cuda), packed


def rel_err(got, want):
    return np.abs(got - want).max() / np.abs(want).max()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("M,K,N", [(1, 768, 2304), (1, 4096, 4096), (3, 576, 960), (4, 1536, 576), (7, 256, 64), (1, 64, 16)])
def test_plain_matmul(cuda, fmt, M, K, N):
    rng = np.random.default_rng(M * 1000 + K + N)
    x, wq, tx, packed = case(rng, M, K, N, fmt, cuda)
    want = x.astype(np.float64) @ wq
    got32 = to_numpy(ops.linear(tx, packed, out_dtype="fp32"))
    assert rel_err(got32, want) < 2e-5, "fp32 accumulation of exact products"
    got16 = to_numpy(ops.linear(tx, packed))
    assert np.array_equal(got16, to_numpy(torch.from_numpy(got32.astype(np.float32)).bfloat16())), "bf16 output is the fp32 one rounded once"


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("M", [1, 2, 4, 6])
def test_rmsnorm_prologue_and_swiglu_epilogue(cuda, fmt, M):
    rng = np.random.default_rng(40 + M)
    K, N = 1024, 2048
    x, wq, tx, packed = case(rng, M, K, N, fmt, cuda)
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, K)).astype(np.float32))
    h = llama.rms(x.astype(np.float64), g, 1e-5)
    gu = h @ wq
    want = llama.glu(gu[:, :N // 2], gu[:, N // 2:])
    got = to_numpy(ops.linear(tx, packed, norm_w=to_bf16_tensor(g, cuda), eps=1e-5, epilogue="swiglu"))
    assert got.shape == (M, N // 2)
    assert rel_err(got, want) < 6e-3, "one bf16 rounding of the output"
    plain = to_numpy(ops.linear(tx, packed, norm_w=to_bf16_tensor(g, cuda), eps=1e-5, out_dtype="fp32"))
    # one token: the norm is applied in fp32 inside the GEMV; more go through the tensor cores, whose operand is the
    # normalised activation rounded to bf16 once (2^-9 relative per element)
    assert rel_err(plain, gu) < (2e-5 if M == 1 else 4e-3)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_residual_epilogue(cuda, fmt):
    rng = np.random.default_rng(7)
    M, K, N = 3, 1536, 576
    x, wq, tx, packed = case(rng, M, K, N, fmt, cuda)
    r = bfp.bf16_round(rng.normal(0, 1, (M, N)).astype(np.float32))
    want = r + x.astype(np.float64) @ wq
    got = to_numpy(ops.linear(tx, packed, epilogue="residual", residual=to_bf16_tensor(r, cuda)))
    assert rel_err(got, want) < 5e-3
    got32 = to_numpy(ops.linear(tx, packed, epilogue="residual", residual=to_bf16_tensor(r, cuda), out_dtype="fp32"))
    assert rel_err(got32, want) < 2e-5


@pytest.fixture
def prefer():
    """fb_linear_prefer for the length of a test (the choice is process-wide)."""
    from ferrite_b200 import _lib
    yield lambda kernel: _lib.lib().fb_linear_prefer(getattr(_lib, "LINEAR_" + kernel))
    _lib.lib().fb_linear_prefer(_lib.LINEAR_AUTO)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("M,K,N,norm,epilogue", [(1, 512, 256, False, "none"), (5, 48, 48, False, "none"), (8, 4096, 6144, True, "none"),
                                                 (9, 1024, 2048, True, "swiglu"), (16, 2048, 1024, False, "residual"),
                                                 (17, 512, 1088, False, "none"), (32, 4096, 4096, True, "swiglu"),
                                                 (32, 14336, 512, False, "residual")])
def test_register_fed_kernel_every_shape_it_takes(cuda, prefer, fmt, M, K, N, norm, epilogue):
    # fb_linear chooses this kernel for 2..8 rows of the smaller matrices only; asked for by name it takes up to 32 rows,
    # one too: 1, 2 and 4 token tiles, K slices over a cluster, a CTA whose second column group does not exist
    # (N = 48, 1088), every epilogue - against exact products, and against the tcgen05 kernel on the same inputs
    rng = np.random.default_rng(M + K + N)
    x, wq, tx, packed = case(rng, M, K, N, fmt, cuda)
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, K)).astype(np.float32)) if norm else None
    r = bfp.bf16_round(rng.normal(0, 1, (M, N)).astype(np.float32)) if epilogue == "residual" else None
    h = llama.rms(x.astype(np.float64), g, 1e-5) if norm else x.astype(np.float64)
    want = h @ wq
    if epilogue == "swiglu":
        want = llama.glu(want[:, :N // 2], want[:, N // 2:])
    if epilogue == "residual":
        want = want + r
    kw = dict(out_dtype="fp32", norm_w=to_bf16_tensor(g, cuda) if norm else None, eps=1e-5, epilogue=epilogue,
              residual=to_bf16_tensor(r, cuda) if r is not None else None)
    prefer("MMA")
    got = ops.linear(tx, packed, **kw)
    again = ops.linear(tx, packed, **kw)
    prefer("TCGEN05")
    other = to_numpy(ops.linear(tx, packed, **kw))
    assert torch.equal(got, again), "the K slices are added in a fixed order"
    got = to_numpy(got)
    tol = 4e-3 if norm else 2e-5  # with a norm the operand is the normalised activation rounded to bf16 once
    assert rel_err(got, want) < tol
    assert rel_err(got, other) < (tol if M > 1 else 4e-3)


def test_register_fed_kernel_beyond_its_one_multiply_scale(cuda, prefer):
    # shared exponents above 187 (values of 2^54 and more) take the two-multiply route; tiny runs next to them too
    rng = np.random.default_rng(3)
    x, wq, tx, packed = case(rng, 8, 512, 256, "bfp8", cuda, sigma=2.0 ** 60)
    prefer("MMA")
    got = to_numpy(ops.linear(tx, packed, out_dtype="fp32"))
    assert rel_err(got, x.astype(np.float64) @ wq) < 2e-5


def test_bfp_matmul_equals_the_matmul_by_its_values(cuda):
    # the reference's claim for a block-float B (test/test_sim.py:373-377): the same result as the matmul by the
    # values it holds; here: quantising the dequantised weight again changes no output bit
    rng = np.random.default_rng(5)
    for fmt in ("bfp8", "bfp4"):
        x, wq, tx, packed = case(rng, 2, 768, 256, fmt, cuda)
        again = ops.quantize(ops.dequantize(packed)[0].contiguous(), fmt)
        assert torch.equal(ops.linear(tx, packed, out_dtype="fp32"), ops.linear(tx, again, out_dtype="fp32"))


def test_misuse_is_refused(cuda):
    x = torch.zeros(1, 64, dtype=torch.bfloat16, device=cuda)
    w = ops.quantize(torch.zeros(64, 48, dtype=torch.bfloat16, device=cuda), "bfp8")
    with pytest.raises(AssertionError):
        ops.linear(x, w, epilogue="swiglu")  # 48 columns do not pair up in runs of 16
    with pytest.raises(AssertionError):
        ops.linear(x, w, epilogue="residual")  # no residual given


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("M,K,N,norm,epilogue", [(1, 512, 256, False, "none"), (8, 4096, 6144, True, "none"), (32, 4096, 4096, False, "residual"),
                                                 (32, 4096, 14336, True, "swiglu"), (17, 512, 1088, False, "none"), (128, 2048, 4096, True, "swiglu"),
                                                 (48, 1088, 384, False, "residual"), (32, 14336, 512, False, "residual")])
def test_persistent_kernel(cuda, prefer, fmt, M, K, N, norm, epilogue):
    # the tcgen05 path as one persistent CTA per SM: runs that are a tail of one tile, whole tiles and a head of another,
    # tiles shared by up to eight CTAs and summed through the workspace in CTA order (so twice the same bits), a tile
    # whose second column group does not exist (N = 1088), K that ends inside a step (1088) - against exact products
    rng = np.random.default_rng(M + K + N)
    x, wq, tx, packed = case(rng, M, K, N, fmt, cuda)
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, K)).astype(np.float32)) if norm else None
    r = bfp.bf16_round(rng.normal(0, 1, (M, N)).astype(np.float32)) if epilogue == "residual" else None
    h = llama.rms(x.astype(np.float64), g, 1e-5) if norm else x.astype(np.float64)
    want = h @ wq
    if epilogue == "swiglu":
        want = llama.glu(want[:, :N // 2], want[:, N // 2:])
    if epilogue == "residual":
        want = want + r
    kw = dict(out_dtype="fp32", norm_w=to_bf16_tensor(g, cuda) if norm else None, eps=1e-5, epilogue=epilogue,
              residual=to_bf16_tensor(r, cuda) if r is not None else None)
    prefer("PERSISTENT")
    got = ops.linear(tx, packed, **kw)
    again = ops.linear(tx, packed, **kw)
    assert torch.equal(got, again), "shared tiles are added in a fixed order"
    assert rel_err(to_numpy(got), want) < (4e-3 if norm else 2e-5)
    from ferrite_b200._lib import lib
    assert lib().fb_status_word() == 0, "no wait gave up"


def test_a_workspace_the_caller_never_zeroed(cuda):
    # the kernels that count in the workspace's head (here the persistent one: 150 tiles, at least one per SM) need it
    # zero; fb_linear zeroes the head of a buffer it has not been given before, so a fresh allocation full of ones works
    from ferrite_b200._lib import lib
    rng = np.random.default_rng(11)
    M, K, N = 32, 512, 19200
    x, wq, tx, packed = case(rng, M, K, N, "bfp8", cuda)
    want = x.astype(np.float64) @ wq
    ws = torch.full((int(lib().fb_linear_workspace_bytes(M, K, N)),), 255, dtype=torch.uint8, device=cuda)
    got = ops.linear(tx, packed, out_dtype="fp32", workspace=ws)
    assert rel_err(to_numpy(got), want) < 2e-5
    assert torch.equal(ops.linear(tx, packed, out_dtype="fp32", workspace=ws), got) and lib().fb_status_word() == 0


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("K,N,norm,epilogue", [(4096, 6144, True, "none"), (4096, 4096, False, "residual"), (4096, 28672, True, "swiglu"),
                                               (14336, 4096, False, "residual"), (100, 64, False, "none"), (64, 64, True, "none"),
                                               (768, 2048, True, "swiglu"), (2048, 1536, False, "none"), (1024, 32064, True, "none"),
                                               (192, 128, False, "swiglu")])
def test_streaming_gemv(cuda, prefer, fmt, K, N, norm, epilogue):
    # one token through the persistent kernel: stretches of units that end inside a column group, groups shared by up to
    # eight CTAs and added in CTA order (twice the same bits), a gate group and its up group finished by whichever CTA
    # arrives last, K that ends inside a unit (100), a matrix of one unit, one CTA for a whole small matrix - against
    # exact products and against the CTA-per-16-columns GEMV
    rng = np.random.default_rng(K + N)
    x, wq, tx, packed = case(rng, 1, K, N, fmt, cuda)
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, K)).astype(np.float32)) if norm else None
    r = bfp.bf16_round(rng.normal(0, 1, (1, N)).astype(np.float32)) if epilogue == "residual" else None
    h = llama.rms(x.astype(np.float64), g, 1e-5) if norm else x.astype(np.float64)
    want = h @ wq
    if epilogue == "swiglu":
        want = llama.glu(want[:, :N // 2], want[:, N // 2:])
    if epilogue == "residual":
        want = want + r
    kw = dict(norm_w=to_bf16_tensor(g, cuda) if norm else None, eps=1e-5, epilogue=epilogue, residual=to_bf16_tensor(r, cuda) if r is not None else None)
    prefer("GEMV_STREAM")
    got = ops.linear(tx, packed, out_dtype="fp32", **kw)
    again = ops.linear(tx, packed, out_dtype="fp32", **kw)
    assert torch.equal(got, again), "shared groups are added in a fixed order, and the counters are back at zero"
    assert rel_err(to_numpy(got), want) < 2e-5
    got16 = ops.linear(tx, packed, **kw)
    assert torch.equal(got16, got.bfloat16()), "bf16 output is the fp32 one rounded once"
    prefer("GEMV")
    plain = ops.linear(tx, packed, out_dtype="fp32", **kw)
    assert rel_err(to_numpy(got), to_numpy(plain).astype(np.float64)) < 2e-5
    from ferrite_b200._lib import lib
    assert lib().fb_status_word() == 0, "no wait gave up"


def test_streaming_gemv_refuses_what_it_does_not_take(cuda, prefer):
    rng = np.random.default_rng(0)
    x, wq, tx, packed = case(rng, 1, 256, 48, "bfp8", cuda)  # N is not a multiple of 64
    want = x.astype(np.float64) @ wq
    assert rel_err(to_numpy(ops.linear(tx, packed, out_dtype="fp32")), want) < 2e-5, "the plain GEMV takes it"
    prefer("GEMV_STREAM")
    with pytest.raises(Exception, match="streaming"):
        ops.linear(tx, packed)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("M,K,N,N2", [(32, 4096, 4096, 2048), (9, 1024, 512, 256), (128, 512, 1088, 128), (33, 14336, 4096, 512)])
def test_norm_handed_from_one_matmul_to_the_next(cuda, fmt, M, K, N, N2):
    # x1 = r + x @ W1; y = silu-less next matmul of rms(x1) * g: the first matmul leaves bf16(x1 * g) and the rows' sums of
    # squares in parts (one per CTA), the second scales its accumulators by them - against the oracle, and against the
    # same two matmuls with the norm as fb_linear's own prologue (the same x1 bit for bit; y within a rounding of fp32 sums)
    rng = np.random.default_rng(M + K + N)
    x, w1, tx, p1 = case(rng, M, K, N, fmt, cuda)
    w2 = bfp.bf16_round(rng.normal(0, 0.02, (N, N2)).astype(np.float32))
    p2 = ops.quantize(to_bf16_tensor(w2, cuda), fmt)
    r = bfp.bf16_round(rng.normal(0, 1, (M, N)).astype(np.float32))
    g = bfp.bf16_round(rng.normal(1, 0.1, (1, N)).astype(np.float32))
    tr, tg = to_bf16_tensor(r, cuda), to_bf16_tensor(g, cuda)
    x1_plain = ops.linear(tx, p1, epilogue="residual", residual=tr)
    y_plain = ops.linear(x1_plain, p2, norm_w=tg, eps=1e-5, out_dtype="fp32")
    x1, xn, sumsq, parts = ops.linear_chained(tx, p1, epilogue="residual", residual=tr, next_norm_w=tg)
    assert parts == ops.chain_parts(p1, M, "residual") and sumsq.shape == (parts, M)
    assert torch.equal(x1, x1_plain), "the handed-on norm does not change the matmul's own result"
    x1f = x1.float()
    assert torch.equal(xn, (x1f * tg.float()).bfloat16()), "xn is bf16(x1 * g)"
    assert torch.allclose(sumsq.sum(0), (x1f * x1f).sum(1), rtol=1e-5)
    y = ops.linear_chained(xn, p2, out_dtype="fp32", eps=1e-5, norm_in=(sumsq, parts))
    want = llama.rms(to_numpy(x1), g, 1e-5) @ bfp.bfp(w2, fmt)
    assert rel_err(to_numpy(y), want) < 4e-3
    assert rel_err(to_numpy(y), to_numpy(y_plain)) < 1e-5
