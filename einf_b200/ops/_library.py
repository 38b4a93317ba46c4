"""Load the built kernel libraries through ctypes and bind their launchers."""
from __future__ import annotations

import ctypes
import threading
from typing import Sequence

from . import build

_libraries: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()

# Which source file holds which launcher.
LAUNCHERS = {
    "einf_embed": "pointwise",
    "einf_add_rmsnorm": "pointwise",
    "einf_rope_kv_write": "pointwise",
    "einf_silu_mul": "pointwise",
    "einf_advance_decode": "pointwise",
    "einf_add_bias": "pointwise",
    "einf_zero_fresh_state": "pointwise",
    "einf_paged_attention_generic": "attention_generic",
    "einf_gemm_simt": "gemm_simt",
    "einf_gemm_tcgen05": "gemm_tcgen05",
    "einf_gemm_tcgen05_splits": "gemm_tcgen05",
    "einf_paged_decode_attention": "attention_bf16",
    "einf_paged_decode_attention_cluster": "attention_bf16",
    "einf_paged_prefill_attention": "attention_bf16",
    "einf_paged_prefill_attention_tcgen05": "attention_tcgen05",
    "einf_paged_decode_attention_tcgen05": "attention_tcgen05",
    "einf_paged_prefill_attention_tcgen05_max_clusters": "attention_tcgen05",
    "einf_paged_decode_attention_tcgen05_max_clusters": "attention_tcgen05",
    "einf_argmax": "sampling",
    "einf_sample": "sampling",
    "einf_report": "sampling",
}


class KernelLibraryError(RuntimeError):
    """A kernel library could not be built or loaded: there is no fallback."""


def library(name: str) -> ctypes.CDLL:
    lib = _libraries.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _libraries.get(name)
        if lib is None:
            try:
                path = build.build_kernel_library(name)
                lib = ctypes.CDLL(str(path))
            except (build.BuildError, OSError) as error:
                raise KernelLibraryError(
                    f"the CUDA kernel library '{name}' is not available and there is no "
                    f"fallback path: {error}"
                ) from error
            _libraries[name] = lib
    return lib


def ensure_built(names: Sequence[str]) -> None:
    """Compile the named libraries side by side and load them."""
    missing = [n for n in dict.fromkeys(names) if n not in _libraries]
    if not missing:
        return
    try:
        build.build_kernel_libraries(missing)
    except build.BuildError as error:
        raise KernelLibraryError(str(error)) from error
    for name in missing:
        library(name)


def launcher(symbol: str, argtypes: Sequence[type], variant: str = "") -> "ctypes._CFuncPtr":
    """Bind ``symbol``; ``variant`` (``MACRO=value``) picks a specialised build of its source."""
    source = LAUNCHERS[symbol] + (f":{variant}" if variant else "")
    function = getattr(library(source), symbol)
    function.argtypes = list(argtypes)
    function.restype = ctypes.c_int
    return function
