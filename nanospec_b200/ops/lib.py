"""Loads the native library and declares its C entry points.

There is one execution path: the CUDA kernels of `csrc/`.  If the library cannot be built
or loaded, or no CUDA device is present, the first kernel call raises; nothing falls back
to the CPU or to a library implementation.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

_lib: ctypes.CDLL | None = None
_path: str | None = None
_launches = 0  # kernel launches made through `call` (graph replays are counted by their owner)


class KernelError(RuntimeError):
    """A native entry point refused its arguments or a CUDA call failed."""


_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

_SIGNATURES: dict[str, list] = {
    "ns_embed": [_P, _P, _P, _I, _I, _I, _I, _P],
    "ns_take_ids": [_P, _P, _P, _P, _I, _P],
    "ns_add_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _P],
    "ns_residual_add": [_P, _P, _I, _I, _I, _P],
    "ns_swiglu": [_P, _P, _I, _I, _I, _I, _P],
    "ns_gemm_f32": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "ns_rope_kv_write": [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "ns_attention_generic": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "ns_sample_rows": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "ns_attention_decode": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "ns_attention_decode_tma": [_P, _I, _P, _P, _L, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P, _P],
    "ns_gemm_bf16_tc_norm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _F, _P, _P, _P, _P, _I, _P, _P],
    "ns_rope_token_kernel_from": [_I],
    "ns_gemm_bf16_tc_rope": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _F, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                             _P, _P],
    "ns_set_pdl": [_I],
    "ns_attention_decode_stages": [_I],
    "ns_gemm_bf16_tc": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "ns_gemm_bf16_tc_gated": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "ns_attention_prefill_tc": [_P, _I, _I, _P, _P, _L, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "ns_wait_probe": [_P, _L, _P, _P],
    "ns_attention_prefill": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P],
}


def load() -> ctypes.CDLL:
    global _lib, _path
    if _lib is not None:
        return _lib
    from ..csrc.build import ensure_built

    path = ensure_built()
    lib = ctypes.CDLL(str(path))
    lib.ns_last_error.restype = ctypes.c_char_p
    lib.ns_last_error.argtypes = []
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue  # declared lazily by `declare` when a newer source adds it
        fn.argtypes = args
        fn.restype = c_int
    _lib, _path = lib, str(path)
    return lib


def declare(name: str, argtypes: list) -> None:
    """Adds or replaces the signature of an entry point (used by modules that own a kernel)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def library_path() -> str | None:
    return _path


def launch_count() -> int:
    return _launches


def call(name: str, *args) -> None:
    global _launches
    lib = load()
    fn = getattr(lib, name, None)
    if fn is None:
        raise KernelError(f"the native library {_path} has no entry point {name}; rebuild it")
    status = fn(*args)
    _launches += 1
    if status != 0:
        raise KernelError(f"{name} failed with status {status}: {lib.ns_last_error().decode(errors='replace')}")
