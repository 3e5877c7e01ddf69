"""The workspace-free decode entry point (nvllm_decode_paged_static).

Some hosts cannot give the library a scratch buffer: the engine has already spent all free
HBM on the KV cache, or it may not call an allocator while it is serving.  For them the
library carries a fixed 32 MiB scratch array of its own.  This file checks that the entry
point gives the same answers as the workspace-taking one, and as the CPU oracle, on two calls
in a row (the second call finds the first call's leftovers in the shared array), that it can
be replayed from a CUDA graph after one eager call, and that it refuses geometries that do
not fit.  It is named to be collected last, so a fail-fast run has already executed
every other test.
"""
import ctypes

import pytest
import torch

from conftest import MAX_ABS_TOL, MEAN_ABS_TOL
from nano_vllm_b200 import _lib, attention as A, workloads as W
from oracle import paged_attention_ref as R

STATIC_BYTES = 32 << 20


def _call_static(lib, dev):
    """Raw C-ABI call: no torch allocation between the arguments and the launch."""
    B, Hq, Hkv, D = dev.geometry
    out = torch.full((B, Hq, D), float("nan"), dtype=torch.bfloat16, device=dev.q.device)
    rc = lib.nvllm_decode_paged_static(
        dev.q.data_ptr(), dev.q.stride(0), dev.k_cache.data_ptr(), dev.v_cache.data_ptr(),
        dev.context_lens.data_ptr(), dev.block_tables.data_ptr(), dev.block_tables.stride(0),
        dev.block_tables.shape[1], out.data_ptr(), out.stride(0), B, Hq, Hkv, D,
        ctypes.c_float(dev.scale), dev.k_cache.shape[0], torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    return out


@pytest.mark.gpu
def test_static_scratch_matches_workspace_entry_point_twice(cuda, lib):
    # two different geometries, both with sequences cut into several partials, so the second call
    # runs over counters and partials that the first one left behind
    cases = [
        W.make_decode_case(41, 6, 1, 1, 16, 8, 128, context_lens=[4000, 3000, 257, 1, 2048, 4096], table_width=16),
        W.make_decode_case(42, 4, 1, 1, 14, 2, 64, context_lens=[700, 5000, 256, 1023], table_width=20),
    ]
    for case in cases:
        dev = case.to(cuda)
        B, Hq, Hkv, D = dev.geometry
        need = _lib.decode_workspace_bytes(B, dev.block_tables.shape[1], Hq, Hkv, D)
        assert 0 < need <= STATIC_BYTES
        expected = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, dev.scale)
        got = _call_static(lib, dev)
        torch.cuda.synchronize()
        diff = (got.float() - expected.float()).abs()
        assert not diff.isnan().any()
        assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL
        ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
        diff = (got.float().cpu() - ref).abs()
        assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL
    # and through the Python wrapper, once more on the last case
    out = torch.empty_like(dev.q)
    A.decode_paged_static(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, dev.scale, out)
    torch.cuda.synchronize()
    assert (out.float() - expected.float()).abs().max().item() <= MAX_ABS_TOL
    assert _lib.read_status() == 0


@pytest.mark.gpu
def test_static_scratch_replayed_from_a_cuda_graph(cuda, lib):
    """One eager call (it looks up the array's address), then the raw C call captured in a graph
    and replayed with other context lengths: the shared array's leftovers must not matter."""
    case = W.make_decode_case(43, 6, 1, 1, 16, 8, 128, context_lens=[4000, 3000, 257, 1, 2048, 4096], table_width=16)
    dev = case.to(cuda)
    _call_static(lib, dev)
    B, Hq, Hkv, D = dev.geometry
    out = torch.zeros((B, Hq, D), dtype=torch.bfloat16, device=cuda)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        rc = lib.nvllm_decode_paged_static(
            dev.q.data_ptr(), dev.q.stride(0), dev.k_cache.data_ptr(), dev.v_cache.data_ptr(),
            dev.context_lens.data_ptr(), dev.block_tables.data_ptr(), dev.block_tables.stride(0),
            dev.block_tables.shape[1], out.data_ptr(), out.stride(0), B, Hq, Hkv, D,
            ctypes.c_float(dev.scale), dev.k_cache.shape[0], torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    for lens in ([4000, 3000, 257, 1, 2048, 4096], [100, 3000, 0, 1, 700, 1500], [3999, 2999, 256, 1, 2047, 4095]):
        dev.context_lens.copy_(torch.tensor(lens, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        expected = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, dev.scale)
        assert (out.float() - expected.float()).abs().max().item() <= MAX_ABS_TOL
    assert _lib.read_status() == 0


def test_static_scratch_refuses_what_does_not_fit(lib):
    """Host-side check, no GPU needed: the size test comes before any device access."""
    B, width, Hq, Hkv, D = 2048, 64, 64, 8, 128
    assert _lib.decode_workspace_bytes(B, width, Hq, Hkv, D) > STATIC_BYTES
    dummy = ctypes.c_void_p(16)
    rc = lib.nvllm_decode_paged_static(dummy, Hq * D, dummy, dummy, dummy, dummy, width, width, dummy, Hq * D,
                                       B, Hq, Hkv, D, ctypes.c_float(0.1), 1000, None)
    assert rc == -4
    assert "built-in array" in _lib.last_error()
