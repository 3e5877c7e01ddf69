"""The C-ABI library: loads without a GPU, exports every declared symbol, and rejects bad
arguments on the host before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

from nano_vllm_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "nvllm_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return re.findall(r"NVLLM_API\s+[\w\s\*]+?\b(nvllm_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(names) == sorted(_lib.SIGNATURES), "ctypes table and header disagree"
    assert lib.nvllm_abi_version() == 2


def test_decode_plan_and_workspace_are_pure_host_arithmetic(lib):
    # work units of 4 warps x 16 tokens (head_dim 128) or 4 x 32 (head_dim 64); the number of thread
    # blocks is a multiple of the KV heads and, without a device, the sizing cap of 1024
    unit, ctas = _lib.decode_plan(256, 16, 16, 8, 128)
    assert unit == 64 and ctas % 8 == 0 and 0 < ctas <= 1024
    unit5, ctas5 = _lib.decode_plan(512, 128, 14, 2, 64)
    assert unit5 == 128 and ctas5 % 2 == 0
    assert _lib.decode_plan(256, 16, 16, 8, 128) == (unit, ctas)
    # 64 KiB of arrival counters + one fp32 partial (D values + max + sum per query head) for each
    # of (1024 / Hkv) ranges + batch pieces; independent of the table width
    ws = _lib.decode_workspace_bytes(256, 16, 16, 8, 128)
    assert ws == 65536 + (1024 // 8 + 256) * 16 * (128 + 2) * 4
    assert _lib.decode_workspace_bytes(256, 64, 16, 8, 128) == ws
    # more (sequence, KV head) pairs than arrival counters
    assert lib.nvllm_decode_workspace_bytes(4096, 16, 16, 8, 128) == -3


def test_empty_batch_is_accepted_by_every_decode_entry_point(lib):
    """Pure host arithmetic: nothing may divide by the batch size."""
    assert _lib.decode_workspace_bytes(0, 16, 16, 8, 128) == 0
    assert _lib.decode_plan(0, 16, 16, 8, 128)[0] == 64
    f = ctypes.c_float(0.1)
    assert lib.nvllm_decode_paged(None, 2048, None, None, None, None, 16, 16, None, 2048, 0, 16, 8, 128, f, 100,
                                  None, 0, None) == 0
    assert lib.nvllm_decode_step(None, 2048, None, 1024, None, 1024, None, None, None, None, None, 16, 16, None, 2048,
                                 0, 16, 8, 128, f, 100, None, 0, None) == 0
    assert lib.nvllm_decode_paged_static(None, 2048, None, None, None, None, 16, 16, None, 2048, 0, 16, 8, 128, f, 100,
                                         None) == 0


@pytest.mark.parametrize("hq,hkv,d,code", [(16, 8, 96, -3), (16, 3, 128, -3), (32, 2, 128, -3), (0, 0, 128, -3)])
def test_unsupported_geometry_is_rejected(lib, hq, hkv, d, code):
    assert lib.nvllm_decode_workspace_bytes(4, 4, hq, hkv, d) == code
    assert _lib.last_error() != ""
    with pytest.raises(_lib.NvllmError):
        _lib.decode_plan(4, 4, hq, hkv, d)


def test_null_and_misaligned_arguments_are_rejected_before_any_launch(lib):
    p16, p8 = ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 8)
    # store: NULL, bad row size, misaligned pointer, stride shorter than the row
    assert lib.nvllm_store_kvcache(None, 1024, p16, 1024, p16, p16, p16, 4, 1024, 256, None) == -1
    assert lib.nvllm_store_kvcache(p16, 1024, p16, 1024, p16, p16, p16, 4, 1020, 256, None) == -3
    assert lib.nvllm_store_kvcache(p8, 1024, p16, 1024, p16, p16, p16, 4, 1024, 256, None) == -2
    assert lib.nvllm_store_kvcache(p16, 512, p16, 1024, p16, p16, p16, 4, 1024, 256, None) == -3
    assert lib.nvllm_store_kvcache(p16, 1028, p16, 1024, p16, p16, p16, 4, 1024, 256, None) == -2
    assert lib.nvllm_store_kvcache(p16, 1024, p16, 1024, p16, p16, p16, 0, 1024, 256, None) == 0  # nothing to do
    # decode: missing workspace
    rc = lib.nvllm_decode_paged(p16, 2048, p16, p16, p16, p16, 16, 16, p16, 2048, 2, 16, 8, 128,
                                ctypes.c_float(0.1), 100, None, 0, None)
    assert rc == -4 and "workspace" in _lib.last_error()
    rc = lib.nvllm_decode_paged(p8, 2048, p16, p16, p16, p16, 16, 16, p16, 2048, 2, 16, 8, 128,
                                ctypes.c_float(0.1), 100, p16, 1 << 30, None)
    assert rc == -2
    # decode step: NULL key, misaligned value stride
    rc = lib.nvllm_decode_step(p16, 2048, None, 1024, p16, 1024, p16, p16, p16, p16, p16, 16, 16, p16, 2048, 2, 16, 8, 128,
                               ctypes.c_float(0.1), 100, p16, 1 << 30, None)
    assert rc == -1
    rc = lib.nvllm_decode_step(p16, 2048, p16, 1024, p16, 1028, p16, p16, p16, p16, p16, 16, 16, p16, 2048, 2, 16, 8, 128,
                               ctypes.c_float(0.1), 100, p16, 1 << 30, None)
    assert rc == -2
    # prefill: NULL cu_seqlens, short stride, paged mode without a table width
    rc = lib.nvllm_prefill_varlen(p16, 2048, p16, 1024, p16, 1024, None, 0, 0, p16, 2048, None, p16, 200, 200, 2, 100, 100,
                                  16, 8, 128, ctypes.c_float(0.1), 0, None)
    assert rc == -1
    rc = lib.nvllm_prefill_varlen(p16, 2048, p16, 512, p16, 1024, None, 0, 0, p16, 2048, p16, p16, 200, 200, 2, 100, 100,
                                  16, 8, 128, ctypes.c_float(0.1), 0, None)
    assert rc == -3
    rc = lib.nvllm_prefill_varlen(p16, 2048, p16, 1024, p16, 1024, p16, 4, 0, p16, 2048, p16, p16, 200, 200, 2, 100, 100,
                                  16, 8, 128, ctypes.c_float(0.1), 10, None)
    assert rc == -3
    assert lib.nvllm_prefill_varlen(p16, 2048, p16, 1024, p16, 1024, None, 0, 0, p16, 2048, p16, p16, 0, 0, 0, 0, 0,
                                    16, 8, 128, ctypes.c_float(0.1), 0, None) == 0  # empty batch


def test_public_header_is_valid_c99_and_cxx():
    """The header is the contract for bindings in any language: it must compile on its own as
    plain C (no C++-isms, no CUDA or torch types) and as C++."""
    import shutil
    import subprocess
    from pathlib import Path
    header = Path(__file__).resolve().parents[1] / "include" / "nvllm_b200.h"
    if not shutil.which("gcc"):
        pytest.skip("no gcc")
    for cmd in (["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c", str(header)],
                ["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", str(header)]):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        assert proc.returncode == 0, proc.stderr


def test_prefill_rejects_more_sequences_than_one_launch_holds(lib):
    """Host-side check before any launch: the persistent kernel keeps its per-sequence tables in
    shared memory, 1024 sequences at most (nano-vllm schedules 512 per step at most)."""
    p16 = ctypes.c_void_p(4096)
    rc = lib.nvllm_prefill_varlen(p16, 2048, p16, 1024, p16, 1024, None, 0, 0, p16, 2048, p16, p16, 4000, 4000, 1025, 100, 100,
                                  16, 8, 128, ctypes.c_float(0.1), 0, None)
    assert rc == -3 and "1024" in _lib.last_error()
