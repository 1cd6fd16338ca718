"""Re-binding a bound method so that one global function it calls gets its result wrapped.

Interface of quarot/monkeypatch.py:5-28 (``copy_func_with_new_globals``,
``add_wrapper_after_function_call_in_method``).  The reference uses it to hook RoPE in LLM
attention; for SAM ``get_rope_function_name`` returns None (quarot/model_utils.py:10-14), so it
is never reached, but the entry points are kept for callers that import them.
"""
from types import FunctionType, MethodType


def copy_func_with_new_globals(f, globals=None):
    """Clone function ``f`` so that its free global names resolve in ``globals``."""
    namespace = f.__globals__ if globals is None else globals
    clone = FunctionType(f.__code__, namespace, f.__name__, f.__defaults__, f.__closure__)
    clone.__dict__.update(f.__dict__)
    clone.__doc__ = f.__doc__
    clone.__qualname__ = f.__qualname__
    clone.__module__ = f.__module__
    clone.__kwdefaults__ = dict(f.__kwdefaults__) if f.__kwdefaults__ else None
    clone.__wrapped__ = f
    return clone


def add_wrapper_after_function_call_in_method(module, method_name, function_name, wrapper_fn):
    """Only calls made directly inside ``module.method_name`` are affected: the method is cloned
    with a private copy of its globals in which ``function_name`` is ``wrapper_fn(original)``.
    Returns that wrapper so the caller can configure it."""
    bound = getattr(module, method_name)
    plain = bound.__func__
    patched_globals = {**plain.__globals__}
    wrapped = wrapper_fn(patched_globals[function_name])
    patched_globals[function_name] = wrapped
    setattr(module, method_name, MethodType(copy_func_with_new_globals(plain, patched_globals), module))
    return wrapped
