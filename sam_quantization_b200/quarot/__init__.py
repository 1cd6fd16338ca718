"""Counterpart of the reference's quarot/ directory: same module and function names."""
from .hadamard_utils import (apply_exact_had_to_linear, get_hadK, is_pow2, matmul_hadU,  # noqa: F401
                             matmul_hadU_cuda, random_hadamard_matrix)
from .monkeypatch import add_wrapper_after_function_call_in_method, copy_func_with_new_globals  # noqa: F401
from .rotate_sam import rotate_sam  # noqa: F401
from .utils import ActQuantWrapper, add_actquant, find_qlayers  # noqa: F401
