"""CPU tests of the C-ABI boundary: the library loads, exports every symbol that
include/cfx.h declares, and fails cleanly (status + message, no abort) without a GPU."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    src = open(os.path.join(ROOT, "include", "cfx.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(cfx_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(cfx):
    L = cfx.lib()
    names = header_symbols()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_binding_covers_header(cfx):
    assert set(header_symbols()) <= set(cfx.declared_symbols())


def test_no_torch_types_in_header():
    src = open(os.path.join(ROOT, "include", "cfx.h")).read()
    # (the word itself appears in a field name of cfx_env_view: the env's torches)
    assert "torch::" not in src and "torch/" not in src and "at::" not in src and "std::" not in src


def test_param_count_matches_reference_constants(cfx):
    L = cfx.lib()
    assert L.cfx_param_count(256, 2, 43) == 620588
    assert L.cfx_param_count(256, 3, 43) == 817196
    assert L.cfx_param_count(0, 2, 43) == 0


def test_forward_io_struct_layout(cfx):
    assert C.sizeof(cfx.ForwardIO) == 9 * 8 + 2 * 8 + 8  # 9 pointers, 2 u64, 2 ints


def test_invalid_arguments_return_status(cfx):
    L = cfx.lib()
    h = C.c_void_p()
    assert L.cfx_policy_create(None, 0, 64, 256, 2, 43, 0) == 1
    assert L.cfx_policy_create(C.byref(h), 0, 48, 256, 2, 43, 0) == 1  # n % 32 != 0
    assert b"multiple of 32" in L.cfx_last_error()
    assert L.cfx_policy_create(C.byref(h), 0, 64, 100, 2, 43, 0) == 1
    assert L.cfx_policy_create(C.byref(h), 0, 64, 256, 0, 43, 0) == 1
    assert L.cfx_policy_create(C.byref(h), 0, 64, 256, 2, 43, 9) == 1
    assert L.cfx_policy_destroy(None) == 0
    assert L.cfx_policy_forward(None, None, None) == 1
    assert L.cfx_policy_load_cfw1(None, b"/nonexistent") == 1


def test_create_without_gpu_is_an_error_not_a_fallback(cfx):
    if cfx.device_count() > 0:
        return
    L = cfx.lib()
    h = C.c_void_p()
    rc = L.cfx_policy_create(C.byref(h), 0, 64, 256, 2, 43, 0)
    assert rc != 0 and h.value is None
    assert len(L.cfx_last_error()) > 0
    try:
        cfx.expand_obs(np.zeros((32, 996), np.uint8))
    except cfx.CfxError:
        pass
    else:
        raise AssertionError("expand ran without a GPU")


def test_record_write_rejects_a_bad_view_before_touching_the_device(cfx):
    """cfx_record_obs validates its view on the host: no view, no envs, a missing field pointer
    and a misaligned record array are refused with a message, with or without a GPU."""
    import ctypes as C
    lib = cfx.lib()
    buf = (C.c_uint8 * 4096)()
    rec = C.addressof(buf)
    assert lib.cfx_record_obs(0, None, rec, 32, None, None) == 1
    assert b"cfx_record_obs" in lib.cfx_last_error()
    # a view is 4 + 4 (pad) + 8 + 8 + 3 * 8 bytes of header, then 40 field pointers
    view = (C.c_uint64 * 64)()
    C.cast(view, C.POINTER(C.c_int32))[0] = 32          # num_envs
    view[1] = rec                                       # state_base
    view[2] = 1024                                      # state_stride
    assert lib.cfx_record_obs(0, view, rec, 32, None, None) == 1
    assert b"field pointer 0" in lib.cfx_last_error()   # player_position is NULL
    for i in range(6, 6 + 40):
        view[i] = rec
    assert lib.cfx_record_obs(0, view, rec + 2, 32, None, None) == 1
    assert b"aligned" in lib.cfx_last_error()
    assert lib.cfx_record_obs(0, view, rec, 64, None, None) == 1   # more envs than the view has
    assert b"num_envs" in lib.cfx_last_error()
