"""fb_decode_attention_static: decode attention for a caller that can neither pass a workspace nor let the library
allocate one (its scratch is an array inside the library).  Called through the C ABI twice in a row and compared with
fb_decode_attention, which runs the same kernels over a caller's workspace: the outputs must be identical.

Collected last (the file name sorts after the others), so a run that stops at the first failure has already run every
other test."""
import numpy as np
import pytest
import torch

from ferrite_b200 import _lib

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_the_workspace_entry_point_twice(cuda):
    lib = _lib.lib()
    T, H, KV, hd, size = 4, 32, 8, 128, 2200  # long enough for the keys to be split across CTAs: the scratch is really used
    need = lib.fb_decode_attention_workspace_bytes(T, H, KV, hd, size)
    assert 0 < need <= lib.fb_decode_attention_static_max_bytes()
    gen = torch.Generator(device=cuda).manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    base = (torch.arange(T, dtype=torch.int32, device=cuda) * size).contiguous()
    for call in range(2):  # the second call finds the array holding the first call's partial sums
        q = torch.randn(T, H * hd, device=cuda, generator=gen).bfloat16()
        cache = torch.randn(2 * KV, T * size, hd, device=cuda, generator=gen).bfloat16()
        place = torch.randint(size // 2, size, (T,), device=cuda, generator=gen).int()
        ws = torch.empty(need, dtype=torch.uint8, device=cuda)
        want, got = torch.zeros(T, H * hd, dtype=torch.bfloat16, device=cuda), torch.zeros(T, H * hd, dtype=torch.bfloat16, device=cuda)
        _lib.check(lib.fb_decode_attention(q.data_ptr(), T, q.stride(0), H, KV, hd, cache.data_ptr(), cache.shape[1], cache.stride(0), base.data_ptr(),
                                           place.data_ptr(), size, 0, want.data_ptr(), want.stride(0), ws.data_ptr(), need, stream))
        _lib.check(lib.fb_decode_attention_static(q.data_ptr(), T, q.stride(0), H, KV, hd, cache.data_ptr(), cache.shape[1], cache.stride(0),
                                                  base.data_ptr(), place.data_ptr(), size, 0, got.data_ptr(), got.stride(0), stream))
        torch.cuda.synchronize()
        assert want.float().abs().max() > 0 and torch.equal(got, want), f"call {call}: the two entry points run the same kernels, bit for bit"


def test_a_call_beyond_the_built_in_scratch_is_refused(cuda):
    lib = _lib.lib()
    T, H, KV, hd, size = 64, 32, 8, 128, 4096  # 512 groups of heads, each split in two: a little over the array's 8 MiB
    assert lib.fb_decode_attention_workspace_bytes(T, H, KV, hd, size) > lib.fb_decode_attention_static_max_bytes()
    z = torch.zeros(16, dtype=torch.int32, device=cuda)
    rc = lib.fb_decode_attention_static(z.data_ptr(), T, H * hd, H, KV, hd, z.data_ptr(), size, size * hd, z.data_ptr(), z.data_ptr(), size, 0,
                                        z.data_ptr(), H * hd, torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and b"built-in array holds" in lib.fb_last_error()
