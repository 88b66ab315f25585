"""``ctypes`` bindings of the compiled kernel libraries.

Each ``csrc/<name>.cu`` becomes ``lib<name>.so`` with ``extern "C"`` entry points that take
raw device pointers, sizes and a stream and return a status.  ``kernel(name, symbol)`` builds
the library on first use, loads it and returns the typed function.  There is no fallback: if
the library cannot be built or loaded, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Tuple

from . import build

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

STATUS_TEXT = {
    1: "bad argument (a size or option this kernel does not take)",
    2: "launch failed (cudaGetLastError after the launch)",
    3: "unaligned pointer or stride",
    4: "size beyond the stated maximum of this entry point",
    5: "CUDA runtime call failed during set-up",
}

# symbol -> (library, argument types); every function returns int.
SIGNATURES: Dict[str, Tuple[str, list]] = {
    "sharpi_embed_gather": ("elementwise", [P, P, I, P, I, I, I, P]),
    "sharpi_add_rmsnorm": ("elementwise", [P, P, P, F, P, I, I, P, I, P, P]),
    "sharpi_swiglu": ("elementwise", [P, P, P, P, I, I, I, P]),
    "sharpi_add": ("elementwise", [P, P, P, LL, P]),
    "sharpi_timestamp": ("elementwise", [P, I, P]),
    "sharpi_qkv_post": ("rope_kv", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, F, I, P]),
    "sharpi_paged_attention_generic": ("attention_generic", [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P]),
    "sharpi_attention_decode": ("attention_decode", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P]),
    "sharpi_attention_prefill": ("attention_prefill", [P, P, P, P, P, I, I, I, I, I, I, I, I, F, P]),
    "sharpi_attention_prefill_tc": ("attention_prefill_tc", [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P]),
    "sharpi_gemm_nt": ("gemm_generic", [P, I, P, I, P, P, P, P, I, I, I, I, I, P, P, P, P]),
    "sharpi_add_bias": ("elementwise", [P, P, I, I, P]),
    "sharpi_router_top1": ("moe", [P, P, I, I, I, I, P, P, P, P, P, P, P]),
    "sharpi_moe_sort": ("moe", [P, I, I, P, P, P]),
    "sharpi_tc_grouped_gemm": ("tc_gemm", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P]),
    "sharpi_gather_rows_bf16": ("tc_gemm", [P, P, P, I, I, P]),
    "sharpi_dense_rows": ("dense_rows", [P, P, P, P, I, I, I, I, P]),
    "sharpi_argmax_rows": ("sampling", [P, I, I, P, P, P]),
    "sharpi_sample_rows_sliced": ("sampling_sliced", [P, I, I, P, P, P, P, P, P, I, I, P, P]),
    "sharpi_apply_penalties": ("sampling", [P, I, P, P, P, P, P, P, I, P]),
    "sharpi_add_logit_bias": ("sampling", [P, I, P, P, P, I, P]),
    "sharpi_sample_rows": ("sampling", [P, I, I, P, P, P, P, P, P, P, P]),
    "sharpi_sample_rows_no_alloc": ("sampling", [P, I, I, P, P, P, P, P, P, P]),
}

_libs: Dict[str, ctypes.CDLL] = {}
_funcs: Dict[str, ctypes._CFuncPtr] = {}
loaded_libraries: Dict[str, str] = {}


class KernelError(RuntimeError):
    pass


def load_library(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        path = build.build_library(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise KernelError(f"cannot load the compiled kernel library {path}: {exc}") from None
        _libs[name] = lib
        loaded_libraries[name] = path
        _apply_programmatic_launch(lib)
    return lib


_programmatic_launch = True


def _apply_programmatic_launch(lib: ctypes.CDLL) -> None:
    fn = getattr(lib, "sharpi_set_programmatic_launch", None)
    if fn is not None:
        fn.argtypes, fn.restype = [c_int], None
        fn(1 if _programmatic_launch else 0)


def set_programmatic_launch(on: bool) -> None:
    """Whether kernels are launched with programmatic stream serialization (a kernel's set-up may overlap the
    tail of the kernel before it).  One switch for the process: it reaches every kernel library that is
    loaded and every one loaded later."""
    global _programmatic_launch
    _programmatic_launch = bool(on)
    for lib in _libs.values():
        _apply_programmatic_launch(lib)


def register(symbol: str, library: str, argtypes: list) -> None:
    """Declare a further entry point (used by kernel files added later and by tests)."""
    SIGNATURES[symbol] = (library, argtypes)
    _funcs.pop(symbol, None)


def kernel(symbol: str):
    fn = _funcs.get(symbol)
    if fn is None:
        try:
            libname, argtypes = SIGNATURES[symbol]
        except KeyError:
            raise KernelError(f"unknown kernel entry point '{symbol}'") from None
        lib = load_library(libname)
        try:
            fn = getattr(lib, symbol)
        except AttributeError:
            raise KernelError(f"library '{libname}' exports no symbol '{symbol}'") from None
        fn.argtypes = argtypes
        fn.restype = c_int
        _funcs[symbol] = fn
    return fn


launch_count = 0      # entry-point calls since the process started; each launches one or more kernels


def check(status: int, symbol: str) -> None:
    global launch_count
    launch_count += 1
    if status != 0:
        raise KernelError(f"{symbol} failed: {STATUS_TEXT.get(status, f'status {status}')}")


def preload(symbols=None) -> None:
    """Build and load the libraries of the given entry points (all if none are named)."""
    names = sorted({SIGNATURES[s][0] for s in (symbols or SIGNATURES)})
    build.build_all(names)
    for n in names:
        load_library(n)
