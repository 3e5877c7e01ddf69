"""Decode-step inputs in one copy and one launch.

Host mirror of what nano-vllm's ``ModelRunner`` does before it can replay a decode graph:
``prepare_decode`` / ``prepare_block_tables`` / ``prepare_sample``
(nanovllm/engine/model_runner.py:151-159, 218-258: six ``torch.tensor(..., pin_memory=True)
.cuda()`` round trips) and the clear-and-copy of the graph's static tensors in ``run_model``
(model_runner.py:271-282: five ``zero_()`` and five slice copies).  Here the step is packed into
one pinned staging block, copied once, and expanded on the device by
``nvllm_decode_step_inputs`` straight into the static tensors.

Staging block for a batch of n sequences (byte offsets)::

    0            tokens        int64[n]    last token of each sequence
    8n           lens          int32[n]    sequence length (the new token included)
    12n          temperatures  fp32[n]     read by the sampler, not by the kernel
    16n          offsets       int32[n+1]  prefix sum of the block-table lengths
    16n+4(n+1)   blocks        int32[...]  the block tables, concatenated
"""
from __future__ import annotations

from itertools import chain

import numpy as np
import torch

from . import _lib


def layout(n: int) -> dict[str, int]:
    """Byte offsets of the sections of the staging block for n sequences."""
    return {"tokens": 0, "lens": 8 * n, "temperatures": 12 * n, "offsets": 16 * n, "blocks": 16 * n + 4 * (n + 1)}


def staging_bytes(max_bs: int, table_width: int) -> int:
    return layout(max_bs)["blocks"] + 4 * max_bs * table_width


def pack(seqs, buf: np.ndarray, with_temperatures: bool = True, temperatures=None) -> tuple[int, int]:
    """Writes the step of ``seqs`` (objects with ``last_token``, ``num_tokens``, ``block_table``
    and, when ``with_temperatures``, ``temperature``: nanovllm/engine/sequence.py) into ``buf``
    (uint8).  Returns (bytes used, widest block table).  Tensor-parallel worker ranks pass
    ``with_temperatures=False``: the sequences they receive carry no sampling parameters
    (Sequence.__getstate__, sequence.py:74-76) and only rank 0 samples -- unless the caller
    hands the step's ``temperatures`` over as a list (the vocabulary-sharded sampling step)."""
    n = len(seqs)
    off = layout(n)
    counts = [len(s.block_table) for s in seqs]
    total = sum(counts)
    end = off["blocks"] + 4 * total
    if end > buf.size:
        raise ValueError(f"staging block of {buf.size} bytes too small for {n} sequences with {total} blocks")
    buf[off["tokens"]:off["lens"]].view(np.int64)[:] = [s.last_token for s in seqs]
    buf[off["lens"]:off["temperatures"]].view(np.int32)[:] = [s.num_tokens for s in seqs]
    if temperatures is not None:
        buf[off["temperatures"]:off["offsets"]].view(np.float32)[:] = temperatures
    elif with_temperatures:
        buf[off["temperatures"]:off["offsets"]].view(np.float32)[:] = [s.temperature for s in seqs]
    offs = buf[off["offsets"]:off["blocks"]].view(np.int32)
    offs[0] = 0
    np.cumsum(counts, out=offs[1:])
    buf[off["blocks"]:end].view(np.int32)[:] = list(chain.from_iterable(s.block_table for s in seqs))
    return end, max(counts) if counts else 0


class DecodeInputStager:
    """Owns the pinned staging block and its device twin for one model runner."""

    def __init__(self, max_bs: int, table_width: int, device):
        self.max_bs, self.table_width = max_bs, table_width
        nbytes = (staging_bytes(max_bs, table_width) + 15) // 16 * 16
        # two host blocks used in turn, each guarded by the event of its last copy, so that packing
        # a step never overwrites bytes a copy still in flight is reading
        self.host = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.host_np = [h.numpy() for h in self.host]
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.turn = 0
        self.dev = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def stage(self, seqs, graph_bs: int, graph_vars: dict, with_temperatures: bool = True,
              temperatures=None) -> torch.Tensor:
        """Fills rows [0, graph_bs) of ``graph_vars`` (the runner's static input tensors,
        model_runner.py:302-307) for a decode step of ``seqs``; returns the step's temperatures
        as a device tensor.  Everything is enqueued on the current stream."""
        n = len(seqs)
        assert 0 < n <= graph_bs <= self.max_bs
        t = self.turn
        self.turn ^= 1
        self.copied[t].synchronize()  # returns at once unless that block's last copy is still running
        end, widest = pack(seqs, self.host_np[t], with_temperatures, temperatures)
        end = (end + 15) // 16 * 16
        self.dev[:end].copy_(self.host[t][:end], non_blocking=True)
        self.copied[t].record()
        off = layout(n)
        bt = graph_vars["block_tables"]
        assert bt.shape[1] == self.table_width and widest <= self.table_width
        base = self.dev.data_ptr()
        with torch.cuda.device(self.dev.device):
            _lib.check(_lib.load().nvllm_decode_step_inputs(
                base, off["tokens"], off["lens"], off["offsets"], off["blocks"], n, graph_bs, widest, self.table_width,
                graph_vars["input_ids"].data_ptr(), graph_vars["positions"].data_ptr(),
                graph_vars["slot_mapping"].data_ptr(), graph_vars["context_lens"].data_ptr(), bt.data_ptr(), bt.stride(0),
                torch.cuda.current_stream(self.dev.device).cuda_stream))
        return self.dev[off["temperatures"]:off["offsets"]].view(torch.float32)
