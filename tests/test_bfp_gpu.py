"""Block-float pack / unpack on the GPU, bit for bit against the reference's numpy model
(the shape of the reference's test_bfp, test/test_sim.py:371-388)."""
import numpy as np
import pytest
import torch

from conftest import bits_to_tensor, golden, to_numpy
from ferrite_b200 import ops
from oracle import bfp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
@pytest.mark.parametrize("name", ["spread", "edge", "wide", "weights"])
def test_cast_is_bit_exact_against_reference_vectors(cuda, fmt, name):
    g = golden("bfp.npz")
    bits = g[f"{name}.bits"]
    packed = ops.quantize(bits_to_tensor(bits, cuda), fmt)
    units = -(-bits.shape[0] // 64) * -(-bits.shape[1] // 64)
    assert packed.data.numel() == units * 4 * (1088 if fmt == "bfp8" else 576)  # ferrite's bytes per 1024 values, whole 64 x 64 units
    got = to_numpy(ops.dequantize(packed))[0]
    want = g[f"{name}.{fmt}"]
    assert np.array_equal(got, want), f"{name}: {np.count_nonzero(got != want)} of {want.size} values differ"
    top, sign, mag = (to_numpy(t)[0] for t in ops.unpack_fields(packed))
    wtop, wsign, wmag = bfp.fields(bfp.bf16_floats(bits), fmt)
    assert np.array_equal(top, wtop) and np.array_equal(sign, wsign) and np.array_equal(mag, wmag)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_cast_of_a_batch_and_a_large_matrix(cuda, fmt):
    rng = np.random.default_rng(9)
    x = rng.normal(0, 0.02, (3, 64, 256)).astype(np.float32)
    t = bits_to_tensor(bfp.bf16_bits(x), cuda)
    assert np.array_equal(to_numpy(ops.dequantize(ops.quantize(t, fmt))), bfp.bfp(x, fmt))
    # a 4096 x 4096 weight: quantise-dequantise is idempotent, and a sample of rows matches the oracle
    w = torch.randn(4096, 4096, device=cuda, generator=torch.Generator(device=cuda).manual_seed(1)).mul_(0.02).bfloat16()
    once = ops.dequantize(ops.quantize(w, fmt))[0]
    twice = ops.dequantize(ops.quantize(once.contiguous(), fmt))[0]
    assert torch.equal(once, twice)
    rows = [0, 1, 17, 2048, 4095]
    assert np.array_equal(to_numpy(once[rows]), bfp.bfp(to_numpy(w[rows]), fmt))


def test_misuse_is_refused(cuda):
    x = torch.zeros(8, 40, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(AssertionError):
        ops.quantize(x, "bfp8")  # 40 columns are not runs of 16
