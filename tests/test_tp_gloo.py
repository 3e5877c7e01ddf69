"""Tensor-parallel sharding of the path, world_size 2 over gloo on CPU: each rank takes its
contiguous chunk of query and KV heads (nanovllm/layers/linear.py:141-163 chunks the fused
qkv weight that way), runs the path on its shard with identical metadata, and the
concatenation over ranks equals the unsharded result.  The path itself has no collective;
the all_gather here only assembles the check."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nano_vllm_b200 import workloads as W
from oracle import paged_attention_ref as R


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def shard_decode_case(case, rank, world):
    B, Hq, Hkv, D = case.geometry
    hq, hkv = Hq // world, Hkv // world
    return W.DecodeCase(case.q[:, rank * hq:(rank + 1) * hq].contiguous(),
                        case.k_new[:, rank * hkv:(rank + 1) * hkv].contiguous(),
                        case.v_new[:, rank * hkv:(rank + 1) * hkv].contiguous(),
                        case.k_cache[:, :, rank * hkv:(rank + 1) * hkv].contiguous(),
                        case.v_cache[:, :, rank * hkv:(rank + 1) * hkv].contiguous(),
                        case.context_lens, case.block_tables, case.slot_mapping, case.scale)


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        case = W.make_decode_case(61, 4, 50, 700, 8, 4, 64)           # same seed on every rank
        full = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
        mine = shard_decode_case(case, rank, world)
        out = R.decode_ref(mine.q, mine.k_cache, mine.v_cache, mine.context_lens, mine.block_tables, mine.scale)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out.contiguous())
        ok = torch.allclose(torch.cat(gathered, dim=1), full, atol=1e-6)
        # bytes shard evenly: every rank moves 1/world of the KV bytes
        total = W.decode_bytes(case.context_lens, 8, 4, 64)
        part = W.decode_bytes(mine.context_lens, 8 // world, 4 // world, 64)
        meta = 4 * (4 + sum((int(n) + 255) // 256 for n in case.context_lens))
        ok = ok and (part - meta) * world == total - meta
        if rank == 0:
            result.put(bool(ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_head_sharded_ranks_reassemble_the_unsharded_result():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert result.get(timeout=5) is True


def _handle_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nano_vllm_b200 import allreduce as AR
        from oracle import paged_attention_ref as R
        mine = bytes([rank + 1]) * 64                       # stands for this rank's IPC handle
        every = AR.gather_handles(mine, rank, world, dist)
        ok = every == b"".join(bytes([r + 1]) * 64 for r in range(world))
        # the sum the peer-memory kernel must reproduce: the collective it replaces, on the same data
        xs = [(torch.randn(1000, generator=torch.Generator().manual_seed(r)) * 2).to(torch.bfloat16) for r in range(world)]
        y = xs[rank].to(torch.float32)
        dist.all_reduce(y)
        ok = ok and torch.equal(y.to(torch.bfloat16), R.allreduce_ref(xs))
        result.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_ranks_exchange_handles_in_rank_order_and_agree_on_the_sum():
    """Host side of the peer-memory all-reduce, world_size 2 over gloo: every rank ends up with
    all handles in rank order, and the oracle's sum equals the collective it stands in for."""
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_handle_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    got = dict(result.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}


def _lm_head_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        g = torch.Generator().manual_seed(77)                        # same on every rank
        vocab, hidden, rows = 4096, 64, 6
        weight = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16)
        x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
        temps = torch.tensor([0.0, 0.6, 1.0, 0.0, 0.3, 2.0])
        noise = torch.empty(rows, vocab).exponential_(1, generator=g)
        per = vocab // world
        mine = torch.nn.functional.linear(x, weight[rank * per:(rank + 1) * per])   # this rank's slice of the logits
        cand = R.sample_candidates_ref(mine, temps, noise[:, rank * per:(rank + 1) * per], rank * per)
        dist.reduce(cand, dst=0, op=dist.ReduceOp.MAX)                # 8 bytes per row instead of the logits
        if rank == 0:
            want, _ = R.lm_head_sample_ref(x, list(weight.chunk(world, 0)), None, temps, noise)
            result.put(R.sample_unpack_ref(cand).tolist() == want.tolist())
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_vocabulary_sharded_sampling_merges_to_the_unsharded_tokens():
    """The tail of a tensor-parallel step, world_size 2 over gloo: every rank reduces its slice of
    the logits to one packed candidate per row, a MAX reduction merges them, and rank 0 holds the
    tokens that ParallelLMHead's gather + cat followed by the Sampler would have produced
    (nanovllm/layers/embed_head.py:78-87, sampler.py:10-26)."""
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lm_head_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert result.get(timeout=5) is True
