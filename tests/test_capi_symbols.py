"""The C-ABI library builds, loads without a GPU, and exports every symbol include/mxfp4_b200.h declares."""
import ctypes
import os
import re

import pytest

from conftest import PKG_DIR, ROOT


def declared_symbols():
    with open(os.path.join(ROOT, "include", "mxfp4_b200.h")) as f:
        text = f.read()
    return re.findall(r"MXFP4_API\s+[\w\s\*]+?\b(mxfp4_\w+)\s*\(", text)


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("mxfp4_build", os.path.join(PKG_DIR, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return ctypes.CDLL(mod.build())


def test_header_declares_the_boundary():
    names = declared_symbols()
    for must in ("mxfp4_version", "mxfp4_last_error", "mxfp4_device_info", "mxfp4_quantize", "mxfp4_dequantize"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_version_and_argument_validation_without_gpu(lib):
    lib.mxfp4_version.restype = ctypes.c_int
    assert lib.mxfp4_version() >= 100
    i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
    lib.mxfp4_quantize.argtypes = [vp, ci, i64, i64, i64, ci, ci, vp, vp, vp]
    lib.mxfp4_quantize.restype = ci
    # argument checks happen before any CUDA call: odd block, unknown dtype / scale format, null pointers
    assert lib.mxfp4_quantize(None, 0, 4, 64, 64, 31, 0, None, None, None) == -2
    assert lib.mxfp4_quantize(None, 9, 4, 64, 64, 32, 0, None, None, None) == -1
    assert lib.mxfp4_quantize(None, 0, 4, 64, 64, 32, 5, None, None, None) == -1
    assert lib.mxfp4_quantize(None, 0, 4, 64, 64, 32, 0, None, None, None) == -1
    assert lib.mxfp4_quantize(None, 0, 0, 64, 64, 32, 0, None, None, None) == 0      # empty input is a no-op
    buf = ctypes.create_string_buffer(256)
    lib.mxfp4_last_error.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.mxfp4_quantize(None, 0, 4, 64, 64, 31, 0, None, None, None)
    lib.mxfp4_last_error(buf, 256)
    assert b"block_size" in buf.value
