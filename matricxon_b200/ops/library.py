"""Loads the compiled kernel library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded the error says so
and nothing runs (the reference's native ops instead decline by returning None,
app/native/fused_ops.py:130-230, and torch takes over; a GPU engine that fell
back silently would hide a missing build).
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

from matricxon_b200.ops import build as _build


class KernelLibraryError(RuntimeError):
    pass


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES: dict[str, tuple[list, object]] = {
    "mx_last_error_message": ([], ctypes.c_char_p),
    "mx_set_chained_launch": ([I], None),
    "mx_embed": ([P, P, I, P, I, I, I, F, P, P], I),
    "mx_softcap": ([P, L, F, P], I),
    "mx_layernorm": ([P, P, P, P, P, I, I, I, F, P], I),
    "mx_layernorm_sum": ([P, P, P, P, P, P, I, I, I, F, P], I),
    "mx_rope_kv_write": ([P, I, I, P, P, P, P, I, I, I, I, I, I, L, I, P, P], I),
    "mx_rope_kv_write_bias": ([P, I, I, P, P, P, P, I, I, I, I, I, I, L, I, P, P, P], I),
    "mx_epilogue": ([P, I, P, P, P, I, L, I, I, P], I),
    "mx_gemm_simt": ([P, P, I, P, P, P, I, I, I, I, I, I, I, I, P], I),
    "mx_gemm_tcgen05": ([P, P, P, P, P, I, I, I, I, I, I, I, I, P, P], I),
    "mx_gemm_tcgen05_force_tiles": ([I], I),
    "mx_gemm_stream": ([P, P, P, P, P, I, I, I, I, I, I, I, I, P, P], I),
    "mx_gemm_skinny": ([P, P, P, P, P, I, I, I, I, I, I, I, I, P], I),
    "mx_gemm_skinny_rope": ([P, P, P, P, I, I, I, I, I, P, P, P, P, L, I, I, I, I, P, P], I),
    "mx_attention_scratch_bytes": ([I, I, I, I], L),
    "mx_paged_attention_mma": ([P, I, P, L, I, P, I, P, P, P, I, I, I, I, I, I, I, F, P, I, I, P, P, P], I),
    "mx_paged_attention_tc": ([P, I, P, L, I, P, I, P, P, P, I, I, I, I, I, I, F, P, I, P, P], I),
    "mx_paged_attention_tc_split": ([P, I, P, L, I, P, I, P, P, P, I, I, I, I, I, I, F, P, I, I, P, P, P], I),
    "mx_paged_attention": ([P, I, I, P, L, I, P, I, P, P, I, I, I, I, I, F, P, I, I, P, P, P], I),
}


def library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = _build.build()
        except _build.BuildError as exc:
            raise KernelLibraryError(
                f"the CUDA kernel library is missing and could not be built: {exc}") from exc
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelLibraryError(f"cannot load {path}: {exc}") from exc
        for name, (argtypes, restype) in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as exc:
                raise KernelLibraryError(f"{path} lacks the entry point {name}") from exc
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
        return lib


def register_signature(name: str, argtypes: list, restype=c_int) -> None:
    """Declares one more entry point (kernel files added later list theirs here)."""
    _SIGNATURES[name] = (argtypes, restype)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def check(code: int, what: str) -> None:
    if code == 0:
        return
    message = library().mx_last_error_message().decode("utf-8", "replace")
    if code == -1:
        raise KernelLibraryError(f"{what}: unsupported size: {message}")
    raise KernelLibraryError(f"{what}: failed with code {code}: {message}")
