"""The C-ABI library loads and exports every function declared in include/*.h (no compute
calls: this runs without a GPU), and the ctypes binding lists the same functions."""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "warpconvnet_b200", "csrc", "libwcn_b200.so")


def declared_functions():
    names = []
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
        names += re.findall(r"\b(wcn_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def lib():
    if not os.path.isfile(LIB):
        from warpconvnet_b200.csrc import build
        build.build()
    return ctypes.CDLL(LIB)


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("wcn_hash_build", "wcn_hash_search", "wcn_unique_mark", "wcn_unique_emit", "wcn_kmap_search",
                 "wcn_kmap_scan", "wcn_kmap_compact", "wcn_nbr_from_maps", "wcn_nbr_transpose", "wcn_morton20",
                 "wcn_gather_rows", "wcn_scatter_add_rows", "wcn_conv_pack_weight", "wcn_conv_fwd",
                 "wcn_status_string", "wcn_version"):
        assert must in names


def test_library_exports_every_declared_function(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_status_strings_and_version(lib):
    lib.wcn_status_string.restype = ctypes.c_char_p
    assert lib.wcn_version() >= 100
    assert lib.wcn_status_string(0) == b"success"
    seen = {lib.wcn_status_string(c) for c in range(-9, 1)}
    assert len(seen) == 10 and b"unknown status" not in seen
    assert lib.wcn_status_string(-77) == b"unknown status"


def test_host_side_argument_checks_need_no_gpu(lib):
    out = ctypes.c_int64(0)
    assert lib.wcn_hash_table_bytes(ctypes.c_int64(1000), ctypes.byref(out)) == 0 and out.value == 20016
    assert lib.wcn_hash_table_bytes(ctypes.c_int64(0), ctypes.byref(out)) == -5
    assert lib.wcn_kmap_workspace_bytes(ctypes.c_int64(1000), 27, ctypes.byref(out)) == 0 and out.value >= 27 * 4 * 4
    assert lib.wcn_conv_packed_weight_bytes(0, 27, 64, 64, 1, ctypes.byref(out)) == 0 and out.value == 27 * 64 * 64 * 2
    assert lib.wcn_conv_packed_weight_bytes(0, 27, 64, 64, 0, ctypes.byref(out)) == 0 and out.value == 0  # fp32: FP32-pipe kernel
    assert lib.wcn_conv_packed_weight_bytes(2, 27, 3, 20, 1, ctypes.byref(out)) == -4


def test_binding_covers_the_header():
    from warpconvnet_b200 import _native
    bound = set(_native.SIGNATURES) | {"wcn_status_string", "wcn_brick_usable_flag"}  # the two that do not return a status
    assert set(declared_functions()) == bound


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from warpconvnet_b200 import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(_native.NativeLibraryError):
        _native.lib()
