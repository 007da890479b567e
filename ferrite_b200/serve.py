"""The sampling head of a batch of logits on the device: what the reference's server reads back instead of whole rows
(models/serve.py:31-47, pinned by test/test_sim.py:2141-2156).  Only `heads` of the serving layer is provided: the slot
engine, sessions and the HTTP server are host code outside the decode path."""
from .tensor import Tensor


def parts_of(cols, most=4096):
    """The fewest equal parts of a row of `cols` logits that are at most `most` wide (1 when nothing divides it)."""
    for p in range(1, cols // 64 + 1):
        if cols % p == 0 and cols // p <= most:
            return p
    return 1


def heads(logits, t=None, k=64):
    """Each row's head of fp32 logits [rows, vocabulary]: its k largest, largest first, the lower column first among
    equals, and their columns (values, ids); and, given t (a column of each row's 1/temperature, fp32), the log of the
    sum of exp(x t) over the whole row in fp32 (lse).  Two rounds of top-k - the best of each part of the row, then the
    best of those by their labels - so no round looks at more than a few thousand values per row and pick; the sum
    is taken part by part as well (short fp32 sums, then a sum of the parts') about the row's maximum, which the head
    already holds."""
    assert logits.dtype == "fp32" and logits.batch == 1 and k <= 64, "fp32 logits, one matrix, k of at most 64"
    parts = parts_of(logits.cols) if logits.cols >= 2 * 4096 else 1
    if parts > 1:
        best, cols = logits.topk(min(k, logits.cols // parts), parts)
        values, ids = best.topk(k, labels=cols)
    else:
        values, ids = logits.topk(k)
    values, ids = values.realize(), ids.realize()
    if t is None:
        return values, ids
    top = values[:, :, :1]  # the row's maximum
    sums = ((logits.split(parts) - top) * t).exp().sum(2)  # [parts, rows, 1]
    lse = (sums.sum(0).log() + top * t).realize()
    return values, ids, lse
