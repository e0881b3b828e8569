"""Loads the compiled kernel library and declares the C signatures of its entry points.

There is no fallback: if the library cannot be built or loaded, or no CUDA device
is present, the first use raises.  The reference binds its native code with
pybind11 (src/entry.cu:599-625); these kernels take raw device pointers and a
stream, so plain ``ctypes`` is enough and nothing has to be compiled against
torch's headers.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

from . import build as _build


class KernelLibraryError(RuntimeError):
    pass


_P = c_void_p
_SIGNATURES = {
    "cpm_embed_rows": [_P, _P, _P, c_int, c_int, c_float, c_int, _P],
    "cpm_add_rmsnorm": [_P, _P, c_float, _P, c_int, _P, _P, c_int, c_int, c_float, c_int, c_int, _P],
    "cpm_residual_add": [_P, _P, c_float, c_int64, c_int, _P],
    "cpm_silu_mul": [_P, _P, c_int, c_int, c_int, c_int, _P],
    "cpm_gemm_skinny_bf16": [_P, _P, _P, c_int, c_int, c_int, c_float, c_int, _P],
    "cpm_rope_store": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_float, c_int, c_int, c_int, c_int, c_int,
                       c_int, _P],
    "cpm_attention_generic": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_float, c_int, _P],
    "cpm_gemm_f32": [_P, _P, _P, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_float, _P],
    "cpm_pool_keys": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "cpm_select_blocks": [_P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int, _P],
    "cpm_advance_decode": [_P, _P, _P, _P, _P, _P, c_int, _P],
    "cpm_decode_attention_bf16": [_P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "cpm_decode_attention_rope_bf16": [_P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_float,
                                       _P, c_float, c_int, _P],
    "cpm_prefill_attention_bf16": [_P, _P, _P, _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float,
                                   _P],
    "cpm_listed_attention_bf16": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P,
                                  c_int, c_int, _P],
    "cpm_gemm_bf16_tcgen05": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "cpm_prefill_attention_tcgen05": [_P, _P, _P, _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_float, _P, c_int, _P],
    "cpm_gemm_bf16_tcgen05_pair": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "cpm_listed_attention_tcgen05": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "cpm_sample_rows": [_P, c_int64, c_int, c_int, _P, _P, _P, c_uint64, _P, _P, _P],
}

# source files whose kernels follow page tables; the checked build (CPMCU_CHECK_BOUNDS=1) keeps a record per file
BOUNDS_FILES = ("attention_bf16", "attention_generic", "attention_tcgen05", "elementwise", "sparse")

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None


def library_path() -> Optional[str]:
    return _lib_path


def load() -> ctypes.CDLL:
    """The kernel library, built at the first call if needed."""
    global _lib, _lib_path
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        checked = os.environ.get("CPMCU_CHECK_BOUNDS", "0") not in ("", "0")
        try:
            path = _build.build(check_bounds=checked)
        except _build.BuildError as e:
            raise KernelLibraryError(f"the CUDA kernel library could not be built: {e}") from None
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelLibraryError(f"the CUDA kernel library {path} could not be loaded: {e}") from None
        lib.cpm_set_pdl.argtypes = [c_int]
        lib.cpm_set_pdl.restype = None
        if os.environ.get("CPMCU_PDL") is not None:      # a mask over the kernel classes; 0 switches it off
            lib.cpm_set_pdl(int(os.environ["CPMCU_PDL"]))
        lib.cpm_set_skinny_prefetch_lines.argtypes = [c_int]
        lib.cpm_set_skinny_prefetch_lines.restype = None
        if os.environ.get("CPMCU_SKINNY_PREFETCH"):
            lib.cpm_set_skinny_prefetch_lines(int(os.environ["CPMCU_SKINNY_PREFETCH"]))
        for name in ("cpm_page_tokens", "cpm_prefill_attention_tile_rows"):
            getattr(lib, name).argtypes = []
            getattr(lib, name).restype = c_int
        lib.cpm_set_tcgen05_narrow.argtypes = [c_int]
        lib.cpm_set_tcgen05_narrow.restype = None
        if os.environ.get("CPMCU_TCGEN05_NARROW") is not None:    # 0: every tcgen05 product on 256-row tiles
            lib.cpm_set_tcgen05_narrow(int(os.environ["CPMCU_TCGEN05_NARROW"]))
        lib.cpm_set_decode_early.argtypes = [c_int]
        lib.cpm_set_decode_early.restype = None
        if os.environ.get("CPMCU_DECODE_EARLY") is not None:      # 0: the decode attention waits before it reads anything
            lib.cpm_set_decode_early(int(os.environ["CPMCU_DECODE_EARLY"]))
        lib.cpm_gemm_tcgen05_error.argtypes = []
        lib.cpm_gemm_tcgen05_error.restype = c_int
        lib.cpm_attention_tcgen05_error.argtypes = []
        lib.cpm_attention_tcgen05_error.restype = c_int
        lib.cpm_select_blocks_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        lib.cpm_select_blocks_scratch_floats.restype = c_int64
        lib.cpm_select_blocks_error.argtypes = []
        lib.cpm_select_blocks_error.restype = c_int
        lib.cpm_listed_tile_error.argtypes = []
        lib.cpm_listed_tile_error.restype = c_int
        lib.cpm_listed_attention_tcgen05_max_pages.argtypes = []
        lib.cpm_listed_attention_tcgen05_max_pages.restype = c_int
        lib.cpm_decode_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.cpm_decode_attention_scratch_floats.restype = c_int64
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                raise KernelLibraryError(f"{path} lacks the entry point {name}; rebuild it") from None
            fn.argtypes = argtypes
            fn.restype = c_int
        lib.checked_files = []
        if checked:
            for tu in BOUNDS_FILES:
                err, lim = getattr(lib, f"cpm_bounds_error_{tu}"), getattr(lib, f"cpm_bounds_limit_{tu}")
                err.argtypes, err.restype = [ctypes.POINTER(c_int * 4)], c_int
                lim.argtypes, lim.restype = [c_int], c_int
                lib.checked_files.append((tu, err, lim))
        _lib, _lib_path = lib, path
        return lib


def declare(name: str, argtypes) -> None:
    """Adds an entry point's signature (used by kernels that register themselves)."""
    _SIGNATURES[name] = list(argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = list(argtypes)
        fn.restype = c_int


LAUNCHES = [0]      # kernels of this library launched (or recorded into a graph) so far


def check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status == -1:
        raise ValueError(f"{what}: the kernel does not take these sizes")
    if status < 0:
        raise KernelLibraryError(f"{what}: kernel library status {status}")
    raise KernelLibraryError(f"{what}: CUDA error {status} at launch")
