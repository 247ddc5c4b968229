"""ctypes binding of ``libxllm_kernels.so`` (the sm_100a kernel library).

The kernels expose a plain C ABI (raw pointers + stream), so no torch C++ headers are involved
in building them and any host (Python here, the C++ runtime elsewhere) can launch them.  On a
machine with a GPU the library is mandatory: a missing library raises instead of silently falling
back to PyTorch ops.  Without a GPU (CPU unit tests) the pure-PyTorch references in
``xllm_b200.ops.reference`` are used.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libxllm_kernels.so"


class KernelLibraryMissing(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def have_gpu() -> bool:
    return torch.cuda.is_available()


def load(build_if_missing: bool = True):
    """Return the loaded kernel library (building it in-tree if it is absent or stale)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if build_if_missing and os.environ.get("XLLM_NO_BUILD", "0") != "1":
        try:
            from .. import _build
            _build.build_kernels()
        except Exception as e:  # a box without nvcc still works from a pre-built library
            if not _LIB_PATH.exists():
                raise KernelLibraryMissing(f"cannot build {_LIB_PATH}: {e}") from e
    if not _LIB_PATH.exists():
        raise KernelLibraryMissing(f"{_LIB_PATH} not found; run `python -m xllm_b200._build`")
    lib = _CheckedLibrary(ctypes.CDLL(str(_LIB_PATH)))
    _declare(lib)
    _LIB = lib
    return lib


class _CheckedLibrary:
    """The kernel library behind a gate: an entry point can only be called after its argument types
    were declared.  Without a declaration ctypes would pass Python integers as 32-bit C ints, i.e.
    device pointers cut in half, and the kernel would write through them."""

    def __init__(self, cdll):
        object.__setattr__(self, "_cdll", cdll)
        object.__setattr__(self, "_declared", set())

    def declare(self, name, argtypes, restype):
        fn = getattr(self._cdll, name, None)
        if fn is None:
            return False
        fn.argtypes = argtypes
        fn.restype = restype
        self._declared.add(name)
        return True

    def __getattr__(self, name):
        fn = getattr(self._cdll, name)          # AttributeError when the symbol does not exist
        if name not in self._declared:
            raise RuntimeError(f"{name}: argument types were never declared (ops/_lib.register_signature); "
                               "refusing to call it with default integer conversion")
        return fn


P = ctypes.c_void_p
I = ctypes.c_int
L = ctypes.c_int64
F = ctypes.c_float
U64 = ctypes.c_uint64


def _declare(lib):
    sig = {
        "xllm_rmsnorm": [P, P, P, P, I, I, F, L, L, I, P],
        "xllm_rmsnorm_static_fp8": [P, P, P, P, P, I, I, F, P],
        "xllm_act_and_mul": [P, P, L, I, L, I, P],
        "xllm_rope_kv": [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P],
        "xllm_paged_decode_attn": [P, P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, P],
        "xllm_paged_decode_attn_window": [P, P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, I, P],
        "xllm_attn_merge": [P, P, P, L, I, I, P],
        "xllm_paged_prefill_attn": [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, P],
        "xllm_paged_prefill_attn_tc": [P, L, P, L, L, P, P, L, P, I, P, P, I, I, I, I, I, F, I, P],
        "xllm_fmha_error_status": [],
        "xllm_sample": [P, L, I, I, I, P, P, P, P, P, U64, U64, P],
        "xllm_sample_rows": [P, L, I, I, I, P, P, P, P, P, P, P, P],
        "xllm_top_logprobs": [P, L, I, I, I, I, P, P, P],
        "xllm_rmsnorm_group_fp8": [P, P, P, P, P, I, I, F, L, I, P],
        "xllm_apply_penalties": [P, L, I, I, I, P, P, I, P, P, P, P],
        "xllm_embedding": [P, P, P, L, I, L, L, P],
        "xllm_gather_rows": [P, P, P, L, L, L, P],
        "xllm_block_copy": [P, I, P, I, L, P],
        "xllm_decode_advance": [P, P, P, P, P, I, P, I, I, P],
        "xllm_resolve_placeholders": [P, P, L, L, P],
    }
    for name, args in sig.items():
        lib.declare(name, args, I)
    lib.declare("xllm_decode_attn_workspace_bytes", [I, I, I, I], L)
    _declare_optional(lib)


# (name, argtypes, restype) of entry points added by later kernel files; declared when present.
_OPTIONAL = []


def register_signature(name, argtypes, restype=I):
    _OPTIONAL.append((name, argtypes, restype))
    if _LIB is not None:
        _declare_optional(_LIB)


def _declare_optional(lib):
    for name, args, res in _OPTIONAL:
        lib.declare(name, args, res)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, name: str):
    if rc != 0:
        raise RuntimeError(f"{name} failed with CUDA error {rc}")
