"""Latency of the peer-memory all-reduce next to NCCL's, on the sizes a decode step sums.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 -m nano_vllm_b200.allreduce_bench

One process per GPU.  Each size is timed with CUDA events over ``--iters`` back-to-back calls
after a warm-up (the time of one call = total / iters; max over ranks), once eagerly and once
replayed from a CUDA graph (how the engine's decode step issues them).  Rank 0 prints one JSON
line per size.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .allreduce import PeerAllReduce
from . import _lib


def _time(fn, iters, warm=10):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device="cuda")  # us per call
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _graphed(fn, calls=8):
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(calls):
                fn()
    return g, calls


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ar = PeerAllReduce(rank, world, 8 << 20, wait_ms=20000)
    for rows, hidden in ((16, 1024), (256, 1024), (64, 4096), (256, 4096), (512, 4096)):
        x = (torch.randn(rows, hidden, generator=torch.Generator().manual_seed(rank)) * 0.5).to(torch.bfloat16).cuda()
        y1, y2 = x.clone(), x.clone()
        ar.all_reduce(y1)
        dist.all_reduce(y2)
        torch.cuda.synchronize()
        diff = float((y1.float() - y2.float()).abs().max())
        scratch = x.clone()
        line = {"bytes": x.numel() * 2, "shape": [rows, hidden], "world": world, "max_abs_diff_vs_nccl": diff}
        line["peer_us"] = round(_time(lambda: ar.all_reduce(scratch), args.iters), 2)
        line["nccl_us"] = round(_time(lambda: dist.all_reduce(scratch), args.iters), 2)
        scratch.copy_(x)
        g, calls = _graphed(lambda: ar.all_reduce(scratch))
        line["peer_graph_us"] = round(_time(g.replay, args.iters // calls + 1) / calls, 2)
        scratch.copy_(x)
        g2, calls = _graphed(lambda: dist.all_reduce(scratch))
        line["nccl_graph_us"] = round(_time(g2.replay, args.iters // calls + 1) / calls, 2)
        line["status"] = _lib.read_status()
        if rank == 0:
            print(json.dumps(line), flush=True)
        del g, g2
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
