"""ferrite_b200: the decode hot path of alkinun/ferrite as hand-written sm_100a CUDA behind a C ABI.

`ferrite_b200.tensor` is the drop-in for `ferrite.tensor` (Tensor, jit); `ferrite_b200.ops` are the
kernels one call at a time; the CUDA library under lib/ is the only compute path.
"""
__all__ = ["ops"]
