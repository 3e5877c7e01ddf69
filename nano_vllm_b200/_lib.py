"""ctypes binding of libnvllm_b200.so (declared in include/nvllm_b200.h).

The shared library is the product; there is no other implementation behind these calls.
Loading fails loudly if the library has not been built (``python -m nano_vllm_b200.build``).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_uint64, c_void_p, POINTER
from pathlib import Path

# NVLLM_B200_LIB points the loader at another build of the same library (e.g. one compiled
# with development instrumentation); by default the in-tree build is used.
LIB_PATH = Path(os.environ.get("NVLLM_B200_LIB") or Path(__file__).resolve().parent / "libnvllm_b200.so")

# name -> (restype, argtypes); mirrors include/nvllm_b200.h one to one
SIGNATURES = {
    "nvllm_store_kvcache": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                      c_int64, c_int32, c_int64, c_void_p]),
    "nvllm_decode_paged": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32,
                                     c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_float, c_int64,
                                     c_void_p, c_int64, c_void_p]),
    "nvllm_decode_step": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int64, c_int32, c_int32, c_int32,
                                    c_int32, c_float, c_int64, c_void_p, c_int64, c_void_p]),
    "nvllm_decode_paged_static": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32,
                                            c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_float, c_int64,
                                            c_void_p]),
    "nvllm_decode_workspace_bytes": (c_int64, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "nvllm_decode_plan": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_int32, POINTER(c_int32), POINTER(c_int32)]),
    "nvllm_prefill_varlen": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                       c_int32, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int32,
                                       c_int32, c_int32, c_int32, c_int32, c_int32, c_float, c_int64, c_void_p]),
    "nvllm_qk_norm_rope_store": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float,
                                           c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32,
                                           c_void_p]),
    "nvllm_sample_tokens": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_uint64, c_uint64,
                                      c_void_p, c_int32, c_int32, c_void_p]),
    "nvllm_sample_candidates": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_uint64, c_uint64,
                                          c_int64, c_void_p, c_int32, c_int32, c_void_p]),
    "nvllm_sample_unpack": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p]),
    "nvllm_decode_step_inputs": (c_int32, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "nvllm_ar_handle_bytes": (c_int64, []),
    "nvllm_ar_init": (c_int32, [c_int32, c_int32, c_int64, c_void_p]),
    "nvllm_ar_connect": (c_int32, [c_void_p]),
    "nvllm_ar_max_bytes": (c_int64, []),
    "nvllm_ar_set_wait_ms": (c_int32, [c_int64]),
    "nvllm_ar_allreduce": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p]),
    "nvllm_ar_set_protocol": (c_int32, [c_int32]),
    "nvllm_ar_protocol": (c_int32, [c_int64, c_int32, c_int64, c_int32]),
    "nvllm_ar_shutdown": (c_int32, []),
    "nvllm_ar_emulated_scratch_bytes": (c_int64, [c_int32, c_int64]),
    "nvllm_ar_allreduce_emulated": (c_int32, [c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int32,
                                              c_int32, c_void_p]),
    "nvllm_ar_gemm_tile": (c_int32, [c_int64, c_int64, c_int64, c_int32, c_int64]),
    "nvllm_ar_gemm_allreduce": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                          c_int64, c_void_p]),
    "nvllm_ar_gemm_allreduce_emulated": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                                   c_void_p, c_int64, c_int64, c_int32, c_void_p]),
    "nvllm_selftest_umma": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nvllm_selftest_wait_expiry": (c_int32, [c_void_p, c_void_p]),
    "nvllm_last_error": (c_char_p, []),
    "nvllm_read_status": (c_int32, [POINTER(c_int32)]),
    "nvllm_abi_version": (c_int32, []),
    "nvllm_launch_count": (c_int64, []),
}

_lib = None


class NvllmError(RuntimeError):
    """A C-ABI entry point rejected its arguments (negative return code)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"nvllm_b200 error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Loads the library once and installs the argument types."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m nano_vllm_b200.build` "
                "(there is no fallback implementation)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return load().nvllm_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code < 0:
        raise NvllmError(code, last_error())


def read_status() -> int:
    """Returns and clears the current device's status word (synchronises the device)."""
    out = c_int32(0)
    check(load().nvllm_read_status(ctypes.byref(out)))
    return out.value


def decode_plan(batch: int, max_blocks: int, hq: int, hkv: int, d: int) -> tuple[int, int]:
    """(tokens per work unit, thread blocks per launch on the current device)."""
    unit, ctas = c_int32(0), c_int32(0)
    check(load().nvllm_decode_plan(batch, max_blocks, hq, hkv, d, ctypes.byref(unit), ctypes.byref(ctas)))
    return unit.value, ctas.value


def decode_workspace_bytes(batch: int, max_blocks: int, hq: int, hkv: int, d: int) -> int:
    n = load().nvllm_decode_workspace_bytes(batch, max_blocks, hq, hkv, d)
    check(n)
    return n


def launch_count() -> int:
    return load().nvllm_launch_count()
