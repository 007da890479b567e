"""The C-ABI library loads and exports every symbol include/ferrite_b200.h declares (no GPU needed)."""
import os
import re

from conftest import ROOT
from ferrite_b200 import _lib


def declared():
    text = open(os.path.join(ROOT, "include", "ferrite_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.lib()
    names = declared()
    assert "fb_linear" in names and "fb_quantize" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures without a declaration"


def test_host_side_calls():
    lib = _lib.lib()
    assert lib.fb_version() >= 1
    # ferrite's footprint, 1088 / 576 bytes per 1024 values (ferrite/compiler.py:19-20), in units of 64 x 64
    assert lib.fb_packed_bytes(_lib.BFP8, 64, 64) == 4 * 1088 and lib.fb_packed_bytes(_lib.BFP4, 128, 64) == 8 * 576
    assert lib.fb_packed_bytes(_lib.BFP8, 32, 48) == 4 * 1088, "rows and columns pad to whole units"
    assert lib.fb_packed_bytes(_lib.BFP8, 32, 40) == 0, "columns come in runs of 16"
    # fb_linear's workspace: a zeroed head of 18 KB (arrival words, row scales, counters), then partial tiles and the
    # normalised activations; one row also leaves room for the streaming GEMV's partial sums, a slot per column group
    # and sharing CTA
    head = 18432
    assert lib.fb_linear_workspace_bytes(32, 4096, 4096) >= head + 32 * 4096 * 2
    assert lib.fb_linear_workspace_bytes(1, 4096, 128256) >= head + (128256 // 64) * 2 * 64 * 4


def test_bad_arguments_are_refused_without_a_gpu():
    lib = _lib.lib()
    rc = lib.fb_quantize(_lib.BF16, None, 1, 32, 32, None, None)
    assert rc == -1 and b"block float" in lib.fb_last_error()
    rc = lib.fb_linear(_lib.BFP8, 16, 1, 30, 32, 16, 32, 16, _lib.BF16, 32, None, 1e-5, 0, None, 0, None, 0, None)
    assert rc == -1 and b"multiple of 4" in lib.fb_last_error()
    rc = lib.fb_linear_prefer(7)
    assert rc == -1 and b"unknown kernel" in lib.fb_last_error()
    assert lib.fb_linear_prefer(_lib.LINEAR_AUTO) == 0


def test_new_entry_points_refuse_bad_arguments_without_a_gpu():
    import ctypes
    lib = _lib.lib()
    two = (ctypes.c_void_p * 2)(16, 32)
    rc = lib.fb_peer_reduce_add(two, two, 0, 9, 16, 64, None, 16, None)
    assert rc == -1 and b"up to 8 ranks" in lib.fb_last_error()
    rc = lib.fb_peer_reduce_add(two, two, 0, 2, 16, 60, None, 16, None)
    assert rc == -1 and b"16-byte pieces" in lib.fb_last_error()
    rc = lib.fb_rope_kv_write_packed(_lib.BF16, 16, 1, 256, 2, 1, 64, 16, 16, 64, 8, 16, 16, None, 1e-5, 16, 128, 16, 64, None)
    assert rc == -1 and b"bfp8 or bfp4 cache" in lib.fb_last_error()
    rc = lib.fb_decode_attention_packed(_lib.BFP8, 16, 1, 128, 2, 1, 96, 16, 64, 16, 16, 64, 0, 16, 128, None, 0, None)
    assert rc == -1 and b"64 or 128" in lib.fb_last_error()
    rc = lib.fb_touched(16, 16, 4, 40, 8, 0, 16, 16, None)
    assert rc == -1 and b"up to 32 choices" in lib.fb_last_error()


def test_empty_shapes_need_no_workspace_and_static_attention_refuses_them():
    lib = _lib.lib()
    assert lib.fb_decode_attention_workspace_bytes(0, 8, 2, 128, 64) == 0 and lib.fb_decode_attention_workspace_bytes(4, 8, 0, 128, 64) == 0
    assert lib.fb_attend_workspace_bytes(0, 4, 128, 64) == 0
    rc = lib.fb_decode_attention_static(16, 0, 1024, 8, 2, 128, 16, 64, 8192, 16, 16, 64, 0, 16, 1024, None)
    assert rc == -1 and b"at least one token" in lib.fb_last_error()
    rc = lib.fb_rope_kv_write(16, 1, 256, 2, 1, 48, 16, 16, 48, 8, 16, 16, 16, 1e-5, 16, 96, 16, 64, 64 * 48, None)
    assert rc == -1 and b"multiple of 64" in lib.fb_last_error()
