"""Peer-memory all-reduce: protocol and arithmetic with all ranks emulated by one cooperative
launch on one GPU (bit-exact against the oracle), the bounded wait running out without a fault,
and -- where the machine has two GPUs -- the real thing across two processes."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from nano_vllm_b200 import _lib, allreduce as AR
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
MAX_BYTES = 4 << 20


def _scratch(cuda, world):
    n = _lib.load().nvllm_ar_emulated_scratch_bytes(world, MAX_BYTES)
    return torch.zeros(n, dtype=torch.uint8, device=cuda)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_sum_bit_exactly_call_after_call(cuda, world):
    """Several calls on the same flag / staging area (the two staging buffers alternate), sizes
    from one vector to 4 MiB, with and without a ragged tail; every rank must hold the oracle's sum."""
    scratch = _scratch(cuda, world)
    g = torch.Generator().manual_seed(world)
    for n in [8, 1000, 262144, 1024 * 1024 + 3, 2 * 1024 * 1024, 8, 4096 * 256]:
        xs = [(torch.randn(n, generator=g) * 2).to(torch.bfloat16) for _ in range(world)]
        outs = AR.all_reduce_emulated([x.to(cuda) for x in xs], scratch, MAX_BYTES)
        torch.cuda.synchronize()
        want = R.allreduce_ref(xs)
        for r, o in enumerate(outs):
            assert torch.equal(o.cpu().view(torch.int16), want.view(torch.int16)), f"rank {r}, {n} elements"
    assert _lib.read_status() == 0


@pytest.mark.parametrize("world", [4, 8])
def test_emulated_protocols_interleave(cuda, world):
    """The four protocols in turn on one area (they share flags, call counts and buffers),
    decode-step sizes and ragged ones; every rank must hold the oracle's sum bit for bit."""
    scratch = _scratch(cuda, world)
    g = torch.Generator().manual_seed(10 + world)
    sizes = [256 * 1024, 16 * 1024, 64 * 4096, 256 * 4096, 8 * world, 1000 * 8 + 3, 256 * 1024, 5]
    for i, n in enumerate(sizes * 2 + sizes[:3]):
        proto = (3, 4, 2, 1, 0)[i % 5]
        xs = [(torch.randn(n, generator=g) * 2).to(torch.bfloat16) for _ in range(world)]
        outs = AR.all_reduce_emulated([x.to(cuda) for x in xs], scratch, MAX_BYTES, protocol=proto)
        torch.cuda.synchronize()
        want = R.allreduce_ref(xs)
        for r, o in enumerate(outs):
            assert torch.equal(o.cpu().view(torch.int16), want.view(torch.int16)), f"call {i}, rank {r}, {n} elements"
    assert _lib.read_status() == 0


@pytest.mark.parametrize("protocol", [3, 4])
def test_absent_peer_in_the_two_shot_protocols(cuda, protocol):
    """Rank 2 of 4 never arrives: the waits of the other ranks run out, nothing hangs."""
    import time
    scratch = _scratch(cuda, 4)
    xs = [torch.ones(256 * 1024, dtype=torch.bfloat16, device=cuda) for _ in range(4)]
    t0 = time.time()
    AR.all_reduce_emulated(xs, scratch, MAX_BYTES, absent_rank=2, protocol=protocol)
    torch.cuda.synchronize()
    assert time.time() - t0 < 10
    assert _lib.read_status() & 4, "NVLLM_STATUS_TIMEOUT expected"


@pytest.mark.parametrize("n", [4096, 1024 * 1024 + 8])
def test_absent_peer_times_out_without_hanging(cuda, n):
    """Rank 1 never arrives: the others give up after the clock limit, set the TIMEOUT bit and a
    latch, and later calls return at once instead of waiting again.  Both protocols: flagged
    cells (small tensor) and staging + flags (large tensor)."""
    import time
    scratch = _scratch(cuda, 2)
    xs = [torch.ones(n, dtype=torch.bfloat16, device=cuda) for _ in range(2)]
    t0 = time.time()
    AR.all_reduce_emulated(xs, scratch, MAX_BYTES, absent_rank=1)
    torch.cuda.synchronize()
    first = time.time() - t0
    assert _lib.read_status() & 4, "NVLLM_STATUS_TIMEOUT expected"
    assert first < 10
    t0 = time.time()
    AR.all_reduce_emulated(xs, scratch, MAX_BYTES, absent_rank=1)
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.5, "the latch must keep later calls from waiting"
    _lib.read_status()  # reading clears the word for the tests that follow
    # the context is intact: a fresh area works
    scratch2 = _scratch(cuda, 2)
    outs = AR.all_reduce_emulated(xs, scratch2, MAX_BYTES)
    torch.cuda.synchronize()
    assert all(bool((o == 2).all()) for o in outs) and _lib.read_status() == 0


def test_bad_arguments_are_refused(cuda, lib):
    assert lib.nvllm_ar_allreduce(None, None, 8, None) == -3      # not connected in this process
    assert lib.nvllm_ar_max_bytes() == 0
    assert lib.nvllm_ar_init(0, 1, 1 << 20, None) == -3           # a world of one
    assert lib.nvllm_ar_init(2, 2, 1 << 20, None) == -3
    assert lib.nvllm_ar_connect(None) == -3
    x = torch.zeros(64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(_lib.NvllmError):
        AR.all_reduce_emulated([x, x], torch.zeros(64, dtype=torch.uint8, device=cuda), MAX_BYTES)


WORKER = r"""
import os, sys, json
sys.path.insert(0, %(root)r)
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
from nano_vllm_b200 import _lib, allreduce as AR
from oracle import paged_attention_ref as R
ar = AR.PeerAllReduce(rank, world, 4 << 20)
ok = True
for i, n in enumerate([8, 1000, 262144, 1024 * 1024 + 3, 2 * 1024 * 1024, 8]):
    xs = [(torch.randn(n, generator=torch.Generator().manual_seed(100 * i + r)) * 2).to(torch.bfloat16) for r in range(world)]
    y = xs[rank].cuda()
    ar.all_reduce(y)
    torch.cuda.synchronize()
    ok = ok and torch.equal(y.cpu().view(torch.int16), R.allreduce_ref(xs).view(torch.int16))
# replayed from a CUDA graph, three calls per replay
y = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
g = torch.cuda.CUDAGraph()
s = torch.cuda.Stream()
with torch.cuda.stream(s):
    ar.all_reduce(y.clone())
    torch.cuda.synchronize()
    with torch.cuda.graph(g, stream=s):
        for _ in range(3):
            ar.all_reduce(y)
for _ in range(4):
    y.fill_(1.0)
    g.replay()
    torch.cuda.synchronize()
    ok = ok and bool((y == world ** 3).all())
# the projection fused with its sum, between plain calls and from a graph (integer operands: exact)
def ints(shape, seed):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randint(-1, 2, shape, generator=gen) * (torch.rand(shape, generator=gen) < 0.25)).to(torch.bfloat16)
for i, (m, n, k) in enumerate([(8, 1024, 256), (200, 1024, 320), (256, 4096, 512)]):
    xs = [ints((m, k), 10 * i + r) for r in range(world)]
    ws = [ints((n, k), 10 * i + 5 + r) for r in range(world)]
    want = R.row_parallel_linear_ref(xs, ws)
    x, w = xs[rank].cuda(), ws[rank].cuda()
    out = ar.linear_all_reduce(x, w)
    t = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    ar.all_reduce(t)
    torch.cuda.synchronize()
    ok = ok and torch.equal(out.cpu().view(torch.int16), want.view(torch.int16)) and bool((t == world).all())
g2 = torch.cuda.CUDAGraph()
with torch.cuda.stream(s):
    with torch.cuda.graph(g2, stream=s):
        for _ in range(3):
            ar.linear_all_reduce(x, w, out)
for _ in range(4):
    out.zero_()
    g2.replay()
    torch.cuda.synchronize()
    ok = ok and torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))
status = _lib.read_status()
dist.barrier()
ar.close()
dist.destroy_process_group()
print(json.dumps({"rank": rank, "ok": bool(ok), "status": status}), flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29571", WORLD_SIZE="2", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER % {"root": str(ROOT)}], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    import json
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, err[-3000:]
        d = json.loads([ln for ln in out.splitlines() if ln.startswith("{")][-1])
        assert d["ok"] and d["status"] == 0, d
