"""The C-ABI library: it loads without a GPU driver, exports every symbol the
header declares, and reports errors as codes plus a message."""

import ctypes
import pathlib
import re

import pytest

from mlc_compiler_b200 import build as B
from mlc_compiler_b200 import runtime

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "mlcb.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlcb_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    B.build_shim()
    lib = ctypes.CDLL(str(B.LIB))
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mlcb.h but not exported"
    assert sorted(runtime._SIGNATURES) == names


def test_version_and_error_channel():
    lib = runtime.load_library()
    assert lib.mlcb_version() == 1
    code = lib.mlcb_launch(None, 1, 32, 0, None, 0, 0, 0)
    assert code != 0
    assert lib.mlcb_last_error()  # a message, not a crash


def test_nvrtc_compile_error_carries_the_log():
    lib = runtime.load_library()
    image, size = ctypes.c_void_p(), ctypes.c_size_t()
    log = ctypes.create_string_buffer(4096)
    code = lib.mlcb_compile(b"this is not CUDA;", b"sm_100a", None, 0, ctypes.byref(image),
                            ctypes.byref(size), log, len(log))
    if code == 200001:
        pytest.skip("NVRTC not installed on this machine")
    assert code > 100000 and not image.value
    assert b"error" in log.value.lower()


def test_nvrtc_produces_an_sm100a_image_without_a_gpu():
    src = ('extern "C" __global__ void probe(float* p) '
           '{ p[threadIdx.x] = __int_as_float(0x7f800000); }')
    try:
        image = runtime.compile_source(src, use_cache=False)
    except runtime.BackendError as e:  # pragma: no cover
        pytest.skip(str(e))
    assert image[:4] == b"\x7fELF"
