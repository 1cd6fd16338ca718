"""The C-ABI boundary without a GPU: the shared library loads, exports every function the public
header declares (and nothing the binding expects is missing), and its entry points reject bad
arguments through the status code / error string before any device work."""
import ctypes
import os
import re

from sam_quantization_b200 import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "samq.h")


def header_code():
    """The header with its comments removed (they mention entry points and libraries by name)."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def declared_functions():
    return sorted(set(re.findall(r"\b(samq_[a-z0-9_]+)\s*\(", header_code())))


def test_header_and_binding_list_the_same_entry_points():
    names = declared_functions()
    assert len(names) >= 20
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)


def built_library():
    """Path of libsamq.so, compiled first when a fresh checkout has not built it yet (nvcc cross-
    compiles without a GPU; a few minutes, once)."""
    if not os.path.exists(_lib.LIB_PATH):
        from sam_quantization_b200.build import build_library
        build_library()
    return _lib.LIB_PATH


def test_library_loads_and_exports_every_declared_symbol():
    assert os.path.exists(built_library())
    raw = ctypes.CDLL(_lib.LIB_PATH)                             # no argtypes: the dynamic symbol table only
    for name in declared_functions():
        assert hasattr(raw, name), name
    lib = _lib.load()
    assert lib.samq_version() >= 100
    for name in _lib.EXPORTED_SYMBOLS:
        fn = getattr(lib, name)
        assert fn.argtypes is not None, name                     # the binding gave every entry a signature


def test_no_torch_types_cross_the_boundary():
    """Plain pointers, sizes and scalars only: the header includes no C++ or torch header."""
    text = header_code()
    assert 'extern "C"' in text
    for banned in ("torch", "at::", "c10::", "std::", "#include <cuda", "Tensor"):
        assert banned not in text, banned
    assert set(re.findall(r"#include\s*[<\"]([^>\"]+)[>\"]", text)) <= {"stdint.h", "stddef.h"}


def test_argument_checks_answer_without_a_device():
    """Entry points validate before they launch: a null operand or a bad enum comes back as a
    non-zero status with a message, not as a crash (none of these calls reaches the GPU)."""
    built_library()
    lib = _lib.load()
    assert lib.samq_quant_workspace_bytes(1) >= 4               # per_tensor needs its absmax slot
    assert lib.samq_quant_workspace_bytes(0) == 0
    rc = lib.samq_act_quant_i8(None, _lib.F16, 4, 64, 64, None, None, 0, 0, 8, None, None, None, None, None, 0, None)
    assert rc != 0 and lib.samq_last_error_string() != b""
    rc = lib.samq_act_quant_i8(None, 99, 0, 64, 64, None, None, 0, 0, 8, None, None, None, None, None, 0, None)
    assert rc != 0
    rc = lib.samq_act_quant_i8(None, _lib.F16, 0, 64, 64, None, None, 0, 0, 11, None, None, None, None, None, 0, None)
    assert rc != 0 and b"n_bits" in lib.samq_last_error_string()
