"""Block-float (bfp8 / bfp4) quantisation model, numpy.  Test infrastructure only.

Restates models/gpt2.py:16-32 of the reference (bf16_bits, bf16_floats, bfp):
values are rounded to bf16 (nearest even), then every run of 16 along the last
axis shares its largest biased exponent; each value keeps a sign and a 7-bit
(bfp8) or 3-bit (bfp4) magnitude below that exponent.

`fields` returns the integers a packed buffer has to hold (shared exponent, sign,
magnitude); `values` turns them back into numbers; `bfp` composes the two and is
what the reference calls `gpt2.bfp`.
"""
import numpy as np

RUN = 16  # values that share one exponent (models/gpt2.py:27)


def bf16_bits(a):
    """float -> bf16 bit pattern, round to nearest even (models/gpt2.py:16-18, packer=False)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_floats(bits):
    """bf16 bit pattern -> float32 (models/gpt2.py:19)."""
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def bf16_round(a):
    return bf16_floats(bf16_bits(a))


def fields(a, fmt="bfp8"):
    """(top, sign, mag) of `a` quantised to fmt.

    top:  uint8, shape a.shape[:-1] + (cols/16,)  shared biased exponent of each run
    sign: uint8 0/1, shape of a; 0 wherever mag is 0 (a zero is stored unsigned,
          ferrite/compiler.py:1635,1662)
    mag:  uint8, shape of a; bfp8: 0..127, bfp4: 0..7
    Follows models/gpt2.py:25-31 step by step.
    """
    a = np.asarray(a)
    assert a.shape[-1] % RUN == 0, "runs of 16 along the last axis"
    bits = bf16_bits(a).astype(np.int64)
    sign = bits >> 15
    expo = (bits >> 7) & 255
    mant = (bits & 127) | np.where(expo != 0, 128, 0)  # the hidden one, unless the exponent field is 0
    shape = a.shape[:-1] + (a.shape[-1] // RUN, RUN)
    expo, mant, sign = expo.reshape(shape), mant.reshape(shape), sign.reshape(shape)
    top = expo.max(-1, keepdims=True)
    shift = np.minimum(top - expo, 8)
    if fmt == "bfp8":
        mag = np.minimum((mant + (1 << shift)) >> (shift + 1), 127)  # half up into 7 bits
    elif fmt == "bfp4":
        mag = np.where(shift < 4, np.minimum((mant + (16 << shift)) >> (shift + 5), 7), 0)  # nearest 3 bits, ties up
    else:
        raise ValueError(fmt)
    sign = np.where(mag != 0, sign, 0)
    return top[..., 0].astype(np.uint8), sign.reshape(a.shape).astype(np.uint8), mag.reshape(a.shape).astype(np.uint8)


def values(top, sign, mag, fmt="bfp8"):
    """Numbers the fields stand for, float64: +-mag * 2^(top-133), bfp4's magnitude in bfp8's top three bits
    (models/gpt2.py:31-32)."""
    q = mag.astype(np.float64) * (16.0 if fmt == "bfp4" else 1.0)
    scale = np.repeat(2.0 ** (top.astype(np.int64) - 133), RUN, axis=-1)
    return np.where(sign != 0, -1.0, 1.0) * q * scale


def bfp(a, fmt="bfp8"):
    """The reference's gpt2.bfp(a, dtype): `a` as the block float holds it, float64."""
    return values(*fields(a, fmt), fmt).reshape(np.shape(a))


def bfp_f32(a, fmt="bfp8", chunk=1024):
    """bfp of a big matrix as float32, a thousand rows at a time (as models/llama.py:650-653 does it)."""
    rows = np.asarray(a).reshape(-1, np.shape(a)[-1])
    out = np.concatenate([bfp(rows[i:i + chunk], fmt).astype(np.float32) for i in range(0, len(rows), chunk)])
    return out.reshape(np.shape(a))
