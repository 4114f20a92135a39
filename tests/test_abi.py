"""The C-ABI library builds, loads and exports every symbol include/bsattn.h declares; argument
validation that happens before any CUDA call is checked here (no GPU needed)."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bsattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsa_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert "bsa_attn_fwd" in names and "bsa_tile_lists_build" in names and len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bsattn.h but not exported"


def test_python_binding_covers_the_header(lib):
    from fa2_custom_mask import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_strerror(lib):
    assert lib.bsa_version() == 200
    assert lib.bsa_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert lib.bsa_strerror(code) not in (b"", b"unknown status")
    assert lib.bsa_strerror(-77) == b"unknown status"


def test_list_sizes(lib):
    from fa2_custom_mask import _lib
    s = _lib.ListSizes()
    assert lib.bsa_tile_list_sizes(2, 3, 7, ctypes.byref(s)) == 0
    assert (s.row_ptr, s.col_idx) == (2 * 3 * 7 + 1, 2 * 3 * 7 * 7)
    assert (s.col_ptr, s.row_idx) == (2 * 3 * 7 + 1, 2 * 3 * 7 * 7)
    assert (s.groups, s.meta) == (5 * 42, 8)
    assert lib.bsa_tile_list_sizes(0, 1, 1, ctypes.byref(s)) == -1


def test_shape_and_dtype_checks_come_before_any_cuda_call(lib):
    s4 = (ctypes.c_int64 * 4)(64 * 64, 64 * 64, 64, 1)
    fake = ctypes.c_void_p(0x1000)
    # N not a multiple of 64 / D != 64
    args = [fake, s4, fake, s4, fake, s4, fake, s4, fake, None, fake, fake, 0, 0, 0.125]
    assert lib.bsa_attn_fwd(*args, 0, 1, 1, 63, 64, None, None, None) == -1
    assert lib.bsa_attn_fwd(*args, 0, 1, 1, 64, 128, None, None, None) == -1
    assert lib.bsa_attn_fwd(*args, 7, 1, 1, 64, 64, None, None, None) == -2
    # innermost stride must be 1
    bad = (ctypes.c_int64 * 4)(64 * 64, 64 * 64, 64, 2)
    args2 = [fake, bad] + args[2:]
    assert lib.bsa_attn_fwd(*args2, 0, 1, 1, 64, 64, None, None, None) == -3
    # misaligned base pointer
    args3 = [ctypes.c_void_p(0x1004)] + args[1:]
    assert lib.bsa_attn_fwd(*args3, 0, 1, 1, 64, 64, None, None, None) == -4
    assert lib.bsa_mask_reduce(fake, s4, 1, 1, 100, fake, None, 0, None) == -1
    assert lib.bsa_reorder(fake, fake, s4, fake, 1, 1, 10, 8, 2, 2, 2, 2, None) == -1  # F*H*W != T
    assert lib.bsa_reorder(fake, fake, s4, fake, 1, 1, 8, 8, 2, 2, 2, 3, None) == -2   # elem size
    assert lib.bsa_selftest_bounded_wait(None, None, None) == -4
    bad_out = (ctypes.c_int64 * 4)(64, 64, 8, 2)
    assert lib.bsa_reorder_strided(fake, s4, fake, bad_out, fake, 1, 1, 8, 8, 2, 2, 2, 2, None) == -3
    assert lib.bsa_inv_reorder_strided(fake, s4, fake, s4, fake, None, 1, 1, 8, 8, 2, 2, 2, 2,
                                       None) == -4                                     # inv_orders
