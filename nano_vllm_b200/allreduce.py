"""All-reduce over peer memory for tensor-parallel ranks (one process per GPU, one node).

Host side of ``nvllm_ar_*``: stands where ``dist.all_reduce(y)`` stands in
``RowParallelLinear.forward`` (nanovllm/layers/linear.py:195-199).  ``torch.distributed`` is used
once, to hand every rank's CUDA IPC handle to every other rank; the reduction itself is one
kernel per rank that reads its peers' staging buffers over NVLink.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def gather_handles(handle: bytes, rank: int, world: int, dist=None) -> bytes:
    """Every rank's handle, concatenated in rank order (an object all-gather on the default
    process group; works on any backend)."""
    if dist is None:
        import torch.distributed as dist
    parts: list = [None] * world
    dist.all_gather_object(parts, handle)
    assert parts[rank] == handle and all(isinstance(p, bytes) and len(p) == len(handle) for p in parts)
    return b"".join(parts)


PROTOCOLS = {0: "auto", 1: "cells", 2: "one-shot", 3: "two-shot", 4: "cells-two-shot"}


def protocol_for(nbytes: int, world: int, max_bytes: int, forced: int = 0) -> str:
    """The protocol the kernel picks for a bf16 tensor of ``nbytes`` (pure host arithmetic in the
    library: the same function the kernel evaluates)."""
    return PROTOCOLS[_lib.load().nvllm_ar_protocol(nbytes // 2, world, max_bytes, forced)]


def prefer_peer_kernel(nbytes: int, world: int, max_bytes: int) -> bool:
    """Whether the peer-memory kernel is used instead of the library collective for a tensor of
    ``nbytes``: whenever it fits the staging buffers and is decode-sized (at most 4 MiB: the
    sizes on which the kernel was timed next to NCCL at 2, 4 and 8 ranks); prefill-sized tensors
    are bandwidth-bound and stay with the library."""
    if nbytes <= 0 or (nbytes + 15) // 16 * 16 > max_bytes:
        return False
    return nbytes <= (4 << 20)


class PeerAllReduce:
    """``all_reduce(x)`` sums a contiguous bf16 CUDA tensor over the ranks in place.  Every rank
    must construct it at the same point and make the same calls."""

    def __init__(self, rank: int, world: int, max_bytes: int = 8 << 20, dist=None, wait_ms: int | None = None):
        lib = _lib.load()
        n = lib.nvllm_ar_handle_bytes()
        buf = ctypes.create_string_buffer(n)
        _lib.check(lib.nvllm_ar_init(rank, world, max_bytes, buf))
        handles = gather_handles(buf.raw, rank, world, dist)
        _lib.check(lib.nvllm_ar_connect(handles))
        if wait_ms is not None:
            _lib.check(lib.nvllm_ar_set_wait_ms(wait_ms))
        self.rank, self.world, self.max_bytes, self.forced = rank, world, max_bytes, 0

    def fits(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.data_ptr() % 16 == 0
                and (x.numel() * 2 + 15) // 16 * 16 <= self.max_bytes)

    def preferred(self, x: torch.Tensor) -> bool:
        """``fits(x)`` and ``prefer_peer_kernel`` for its size."""
        return self.fits(x) and prefer_peer_kernel(x.numel() * 2, self.world, self.max_bytes)

    def protocol(self, nbytes: int) -> str:
        return protocol_for(nbytes, self.world, self.max_bytes, self.forced)

    def force_protocol(self, protocol: int) -> None:
        """0 automatic, 1 cells, 2 one shot, 3 two shots, 4 cells in two shots; every rank must set the same."""
        _lib.check(_lib.load().nvllm_ar_set_protocol(protocol))
        self.forced = protocol

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if not self.fits(x):
            raise RuntimeError("PeerAllReduce.all_reduce: contiguous 16-byte-aligned bf16 CUDA tensor of at most "
                               f"{self.max_bytes} bytes expected")
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().nvllm_ar_allreduce(x.data_ptr(), x.data_ptr(), x.numel(),
                                                      torch.cuda.current_stream(x.device).cuda_stream))
        return x

    def linear_fits(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        """Whether ``linear_all_reduce(x, weight)`` can run: 2-D bf16 CUDA operands with 16-byte
        aligned rows and a shape the fused kernel's cell areas hold (decode-sized batches)."""
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and weight.dim() == 2
                and weight.dtype == torch.bfloat16 and x.shape[1] == weight.shape[1]
                and x.stride(1) == 1 and weight.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
            return False
        return _lib.load().nvllm_ar_gemm_tile(x.shape[0], weight.shape[0], x.shape[1], self.world, self.max_bytes) > 0

    def linear_all_reduce(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``all_reduce(F.linear(x, weight))`` as one launch: ``x`` [tokens, in / ranks], ``weight``
        [out, in / ranks] (this rank's shard of a row-parallel projection), result [tokens, out]."""
        if not self.linear_fits(x, weight):
            raise RuntimeError("PeerAllReduce.linear_all_reduce: shape or layout not supported (see linear_fits)")
        m, k = x.shape
        n = weight.shape[0]
        if out is None:
            out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().nvllm_ar_gemm_allreduce(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0),
                                                           out.data_ptr(), out.stride(0), m, n, k,
                                                           torch.cuda.current_stream(x.device).cuda_stream))
        return out

    def close(self) -> None:
        _lib.check(_lib.load().nvllm_ar_shutdown())


def all_reduce_emulated(inputs: list[torch.Tensor], scratch: torch.Tensor, max_bytes: int,
                        absent_rank: int = -1, protocol: int = 0) -> list[torch.Tensor]:
    """All ranks' reductions in one cooperative launch on one device (test aid): returns one
    output per rank.  ``scratch``: uint8, zero-filled before its first use, kept between calls.
    ``protocol``: 0 automatic, 1 cells, 2 one shot, 3 two shots, 4 cells in two shots."""
    world = len(inputs)
    outs = [torch.empty_like(x) for x in inputs]
    arr = ctypes.c_void_p * world
    with torch.cuda.device(inputs[0].device):
        _lib.check(_lib.load().nvllm_ar_allreduce_emulated(
            world, arr(*[x.data_ptr() for x in inputs]), arr(*[o.data_ptr() for o in outs]), inputs[0].numel(),
            scratch.data_ptr(), scratch.numel(), max_bytes, absent_rank, protocol,
            torch.cuda.current_stream(inputs[0].device).cuda_stream))
    return outs


def linear_all_reduce_emulated(xs: list[torch.Tensor], weights: list[torch.Tensor], scratch: torch.Tensor,
                               max_bytes: int, mode: int = 0) -> list[torch.Tensor]:
    """The fused projection + all-reduce of every rank in one cooperative launch on one device
    (test aid): ``xs[r]`` [m, k], ``weights[r]`` [n, k] contiguous; returns one [m, n] output per
    rank.  ``scratch`` as for ``all_reduce_emulated`` (the two may share it).  ``mode``: 0 the
    kernel's choice, 1 one shot (every rank sums every tile), 2 two shots (a tile's owner sums)."""
    world = len(xs)
    m, k = xs[0].shape
    n = weights[0].shape[0]
    outs = [torch.empty(m, n, dtype=torch.bfloat16, device=xs[0].device) for _ in range(world)]
    arr = ctypes.c_void_p * world
    with torch.cuda.device(xs[0].device):
        _lib.check(_lib.load().nvllm_ar_gemm_allreduce_emulated(
            world, arr(*[x.data_ptr() for x in xs]), arr(*[w.data_ptr() for w in weights]),
            arr(*[o.data_ptr() for o in outs]), m, n, k, scratch.data_ptr(), scratch.numel(), max_bytes, mode,
            torch.cuda.current_stream(xs[0].device).cuda_stream))
    return outs
