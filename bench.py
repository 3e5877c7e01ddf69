"""Benchmark of the paged-attention path: paged GQA decode attention, HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: one decode step of one layer in Qwen3-8B geometry (32 query / 8 KV heads, head_dim
128), 256 sequences with context lengths uniform in [2048, 8192], KV cache in 256-token
blocks addressed through a scattered block table.  With N GPUs the heads and the cache are
sharded N ways (tensor parallelism: 32/N query and 8/N KV heads per rank, identical lengths
and tables on every rank); the path has no collective, so ranks only meet at the timing
barrier.  Total work is fixed as N grows ("strong" scaling).

A step = what the attention layer does for that batch: store_kvcache of the new token's K/V
and the paged decode, as ONE launch (attention.decode_step).  `value` counts the step's
algorithmic bytes (every live K/V byte once, q, o, lengths, table entries, the stored rows)
over the device time of K steps with everything resident in HBM; the K-step region is timed
R times and the median is reported.  `e2e` is the same step driven from pinned host buffers
(q, new K/V rows and metadata copied in, output copied out, all inside the timed region).  The
KV cache itself is the path's device-resident state in the engine (it never lives on the
host), so it is not part of the per-step host traffic.  After the timed regions the output of
the very launch that was timed is compared with the CPU oracle on a sample of sequences
(`parity_check`); a mismatch fails the run.

The line ends with the end-to-end metric: output tok/s of the nano-vllm engine with this
package plugged in, and of the stock engine, at tensor-parallel size N (child processes that
start after the ranks of the kernel benchmark have gone).

`--impl reference` times the CPU restatement of the reference path (fp32 torch SDPA over
blocks gathered through the table, oracle/paged_attention_ref.py) on the host cores, on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "paged_decode_attn_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write, from one ncu capture of decode_paged_kernel on the 8-rank shard of this
# workload) per algorithmic byte of the launch; traffic grows in proportion to the KV bytes read.
DECODE_TRAFFIC_PER_ALGO_BYTE = 1.008
CPU_SAMPLE_SEQS = 32        # sequences per step of the reference arm
CPU_BASELINE_SEQS = 128     # sequences in the cpu_baseline leg of our arm (10 passes)
PARITY_SEQS = 8             # sequences of the timed launch that are checked against the oracle
MAX_ABS_TOL, MEAN_ABS_TOL = 2e-2, 2e-3
MIN_TIMED_SECONDS = 0.5     # the K-step region is repeated until this much time has been measured
ENGINE_BUDGET_S = 660       # wall-clock budget of the end-to-end engine runs that close the line


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="sequences in the decode batch")
    ap.add_argument("--shard-of", type=int, default=0, choices=[0, 2, 4, 8],
                    help="with --gpus 1: time rank 0's shard of a run on that many GPUs (profiling aid: the per-rank "
                         "launch of a tensor-parallel run on one GPU)")
    ap.add_argument("--repeats", type=int, default=0, help="timed regions of --steps steps (0: as many as give 0.5 s)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the store/prefill/long-context extras")
    ap.add_argument("--no-engine", action="store_true",
                    help="skip the end-to-end nano-vllm engine runs (output tok/s) that close the line")
    ap.add_argument("--kernel", default=None,
                    choices=["prefill", "prefill_long", "prefill_d64", "store", "decode", "decode_tp8", "decode_engine",
                             "decode_long", "sampler", "allreduce", "gemm_allreduce"],
                    help="time only this kernel and print its line (profiling aid; allreduce and gemm_allreduce run under torchrun)")
    ap.add_argument("--ar-protocol", type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help="with --kernel allreduce: force a protocol (0 automatic, 1 cells, 2 one shot, 3 two shots, "
                         "4 cells in two shots)")
    ap.add_argument("--with-flash-attn", action="store_true",
                    help="with --kernel: also time the library kernels the reference calls (flash-attn, Triton "
                         "store) on the same inputs, if they are importable")
    return ap.parse_args()


def workload_name(n):
    return (f"Qwen3-8B geometry single-layer paged decode step, batch 256, ctx U[2048,8192], block 256, "
            f"TP={n} ({32 // n}q/{8 // n}kv heads per rank, D=128)")


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except Exception:
            pass
    return {}


def hbm_peak():
    pk = measured_peaks()
    if "hbm_gbs" in pk:
        return float(pk["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs: a read+write copy, so a read-mostly kernel can exceed it)"
    return FALLBACK_HBM_GBS, "fallback (MEASURED_PEAKS.json absent)"


# ---- clocks --------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the
    timed regions run; falls back to one nvidia-smi query if NVML is not importable."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, torch_device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self._nv = pynvml
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(torch_device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        if not self.samples:
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=20).stdout.strip().splitlines()[0]
                cur, mx = (int(x) for x in out.split(","))
                self.samples, self.max_mhz = [cur], mx
            except Exception:
                pass
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- the CPU restatement of the reference path -----------------------------------------------

def cpu_sample(case, seqs):
    """Compacts the given sequences (an int = the first n) of a (device) decode case into a small
    host case: only their blocks are kept, renumbered, so the host copy stays small."""
    import torch
    from nano_vllm_b200 import workloads as W
    idx = torch.arange(seqs) if isinstance(seqs, int) else torch.as_tensor(seqs, dtype=torch.int64)
    didx = idx.to(case.q.device)
    lens = case.context_lens[didx].cpu()
    bt = case.block_tables[didx].cpu()
    used = torch.unique(bt[bt >= 0].to(torch.int64))
    remap = torch.full((int(case.k_cache.shape[0]),), -1, dtype=torch.int32)
    remap[used] = torch.arange(used.numel(), dtype=torch.int32)
    new_bt = torch.where(bt >= 0, remap[bt.clamp(min=0).to(torch.int64)], torch.full_like(bt, -1))
    blocks = used.to(case.k_cache.device)
    return W.DecodeCase(case.q[didx].cpu(), case.k_new[didx].cpu(), case.v_new[didx].cpu(),
                        case.k_cache[blocks].cpu(), case.v_cache[blocks].cpu(), lens, new_bt,
                        torch.zeros(idx.numel(), dtype=torch.int32), case.scale)


def parity_against_oracle(case, out, n_seqs=PARITY_SEQS):
    """Compares `out`, the output of a launch over `case` (cache already holding the new tokens),
    with the CPU oracle on n_seqs evenly spaced sequences, all heads of this rank."""
    from oracle import paged_attention_ref as R
    B = case.q.shape[0]
    idx = sorted({int(i * B / n_seqs) for i in range(min(n_seqs, B))})
    host = cpu_sample(case, idx)
    ref = R.decode_ref(host.q, host.k_cache, host.v_cache, host.context_lens, host.block_tables, host.scale)
    diff = (out[idx].float().cpu() - ref).abs()
    mx, mean = float(diff.max()), float(diff.mean())
    ok = bool(math.isfinite(mx) and mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL)
    return {"seqs": len(idx), "tokens": int(host.context_lens.sum()), "max_abs": round(mx, 6), "mean_abs": round(mean, 7),
            "tol": [MAX_ABS_TOL, MEAN_ABS_TOL], "ok": ok}


def use_all_host_threads():
    """The launcher for several ranks exports OMP_NUM_THREADS=1, which would leave the CPU path on
    one thread; give it what a single-process run gets by default (one thread per CPU this
    process may run on)."""
    import torch
    if os.environ.get("OMP_NUM_THREADS") == "1" and hasattr(os, "sched_getaffinity"):
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    return torch.get_num_threads()


def time_cpu_reference(host_case, steps, warmup):
    import torch
    from nano_vllm_b200 import workloads as W
    from oracle import paged_attention_ref as R
    use_all_host_threads()
    B, Hq, Hkv, D = host_case.geometry
    nbytes = W.decode_bytes(host_case.context_lens, Hq, Hkv, D)
    fn = lambda: R.decode_ref(host_case.q, host_case.k_cache, host_case.v_cache, host_case.context_lens,
                              host_case.block_tables, host_case.scale)
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    return nbytes / dt / 1e9, dt, nbytes, torch.get_num_threads()


def run_reference(args):
    """The reference arm: CPU path on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from nano_vllm_b200 import workloads as W
    # same seeded lengths / tables / geometry as the GPU arm, full heads; only the sampled
    # sequences' blocks are materialised (on the host)
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(2048, 8192 + 1, (args.batch,), generator=g)[:CPU_SAMPLE_SEQS].tolist()
    host = W.make_decode_case(4, CPU_SAMPLE_SEQS, 0, 0, 32, 8, 128, device="cpu", context_lens=lens, spare_blocks=2)
    gbs, dt, nbytes, threads = time_cpu_reference(host, args.steps, args.warmup)
    sample = f"first {CPU_SAMPLE_SEQS} of 256 sequences per step ({nbytes / 1e6:.0f} MB algorithmic), full 32q/8kv heads"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(1), "sample": sample},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- our arm -------------------------------------------------------------------------------

def build_once(local_rank, barrier):
    """One rank per node compiles (if the library is stale); the others wait, then load."""
    from nano_vllm_b200 import _lib, build as _build
    if local_rank == 0:
        _build.build()
    barrier()
    _lib.load()


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nano_vllm_b200 import _lib, attention as A, workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert 8 % world == 0, "the 8 KV heads shard over 1, 2, 4 or 8 GPUs"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    build_once(local, barrier)

    shard_of = args.shard_of if world == 1 and args.shard_of else world
    case = W.cfg4_decode(shard_of, rank, dev, batch=args.batch)
    B, Hq, Hkv, D = case.geometry
    lens_host = case.context_lens.cpu()
    decode_bytes_rank = W.decode_bytes(lens_host, Hq, Hkv, D)
    step_bytes_rank = decode_bytes_rank + W.store_bytes(B, Hkv * D)
    out = torch.empty_like(case.q)
    stream = torch.cuda.current_stream()

    def step():
        A.decode_step(case.q, case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping,
                      case.context_lens, case.block_tables, case.scale, out=out)

    def timed_region(fn, steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        barrier()
        return max_over_ranks(a.elapsed_time(b))

    # ---- device-resident timing: R regions of exactly K steps, median
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    probe_ms = timed_region(step, args.steps)
    repeats = args.repeats or max(3, min(200, math.ceil(MIN_TIMED_SECONDS * 1e3 / max(probe_ms, 1e-3))))
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = _lib.launch_count()
    region_ms = [timed_region(step, args.steps) for _ in range(repeats)]
    launches = (_lib.launch_count() - launches0) // repeats
    ms_per_step = statistics.median(region_ms) / args.steps
    status = _lib.read_status()

    # the launch's own duration: a pass with events around every launch (outside the regions above)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for a, b in kev:
        a.record(stream)
        step()
        b.record(stream)
    barrier()
    kernel_ms = max_over_ranks(statistics.median(a.elapsed_time(b) for a, b in kev))

    # ---- end to end from pinned host buffers
    # The step's inputs (q, the new K/V rows, slot ids, lengths, block table) sit in ONE pinned
    # host staging block and go over in one copy; the device tensors are views of its device twin.
    names = ("q", "k_new", "v_new", "slot_mapping", "context_lens", "block_tables")
    offs, total = {}, 0
    for k in names:
        t = getattr(case, k)
        offs[k] = total
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    host_block = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_block = torch.empty(total, dtype=torch.uint8, device=dev)

    def view(block, k):
        t = getattr(case, k)
        n = t.numel() * t.element_size()
        return block[offs[k]:offs[k] + n].view(t.dtype).view(t.shape)

    for k in names:
        view(host_block, k).copy_(getattr(case, k).cpu())
    devbuf = {k: view(dev_block, k) for k in names}
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(getattr(case, k).numel() * getattr(case, k).element_size() for k in names)
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        dev_block.copy_(host_block, non_blocking=True)
        A.decode_step(devbuf["q"], devbuf["k_new"], devbuf["v_new"], case.k_cache, case.v_cache, devbuf["slot_mapping"],
                      devbuf["context_lens"], devbuf["block_tables"], case.scale, out=out)
        out_host.copy_(out, non_blocking=True)
        stream.synchronize()  # the caller reads the result on the host

    def e2e_region(steps):
        barrier()
        w0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        torch.cuda.synchronize()
        return max_over_ranks((time.perf_counter() - w0) * 1e3)

    for _ in range(3):
        e2e_step()
    e2e_regions = [e2e_region(args.steps) for _ in range(repeats)]
    e2e_ms = statistics.median(e2e_regions) / args.steps
    clocks = sampler.stop()

    # ---- is what was timed right?  (outside every timed region)
    step()
    torch.cuda.synchronize()
    parity = parity_against_oracle(case, out)
    parity_e2e_ok = bool(torch.equal(out_host, out.cpu()))
    if world > 1:
        t = torch.tensor([parity["max_abs"], parity["mean_abs"], 0.0 if parity["ok"] and parity_e2e_ok else 1.0],
                         dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity.update(max_abs=round(float(t[0]), 6), mean_abs=round(float(t[1]), 7), ok=bool(t[2] == 0.0))
        parity["ranks"] = world
    parity["e2e_output_identical"] = parity_e2e_ok

    total_bytes = step_bytes_rank * world  # same lengths on every rank, heads split evenly
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9
    peak, peak_src = hbm_peak()
    achieved = decode_bytes_rank / (ms_per_step * 1e-3) / 1e9
    traffic = None if DECODE_TRAFFIC_PER_ALGO_BYTE is None else int(decode_bytes_rank * DECODE_TRAFFIC_PER_ALGO_BYTE)
    unit_tokens, ctas = _lib.decode_plan(B, case.block_tables.shape[1], Hq, Hkv, D)
    mhz = clocks.get("sm_mhz")

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "repeats": repeats, "ms_per_step_min_max": [round(min(region_ms) / args.steps, 4), round(max(region_ms) / args.steps, 4)],
        "ms_x_sm_mhz": round(ms_per_step * mhz, 1) if mhz else None,
        "config": {"workload": workload_name(shard_of) + (f" -- rank 0's shard only, on one GPU" if shard_of != world else ""),
                   "global_batch": B, "kv_bytes_per_step": int(total_bytes),
                   "decode_plan": {"unit_tokens": unit_tokens, "thread_blocks": ctas},
                   "l2": "inputs (KV cache shard) larger than L2, re-read every step; no flush needed",
                   "parallelism": f"tp{world}"},
        "pct_of_nominal_8TBps_per_gpu": round(100 * value / world / NOMINAL_HBM_GBS, 1),
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
                "ms_per_step_min_max": [round(min(e2e_regions) / args.steps, 4), round(max(e2e_regions) / args.steps, 4)],
                "h2d_bytes_per_step": int(h2d * world), "d2h_bytes_per_step": int(d2h * world)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "decode_paged_kernel (store of the new rows and merge of partials inside)",
                     "achieved": round(achieved, 1), "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                     "peak_source": peak_src, "traffic": traffic, "algorithmic_bytes_per_launch": int(decode_bytes_rank),
                     "avg_launch_ms": round(ms_per_step, 4), "launch_alone_ms": round(kernel_ms, 4),
                     "how": "algorithmic bytes of one launch / (timed region / launches in it): launch gaps count against the kernel"},
        "parity_check": parity,
        "device_status_word": status,
    }

    if rank == 0 and world == 1 and shard_of == 1:
        n_cpu = min(B, CPU_BASELINE_SEQS)
        sample_case = cpu_sample(case, n_cpu)
        gbs, dt, nbytes, threads = time_cpu_reference(sample_case, steps=10, warmup=1)
        line["cpu_baseline"] = {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"first {n_cpu} of {B} sequences, 10 timed passes of {dt * 1e3:.0f} ms "
                                          f"({nbytes / 1e6:.0f} MB algorithmic each)"}
        del sample_case
        if not args.no_secondary:
            line["secondary"] = secondary(dev, peak)
    del case, out, dev_block, devbuf
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        if not args.no_engine and shard_of == world:
            line["engine"] = engine_runs(world)
            mine = line["engine"].get("qwen3-0.6b", {}).get("b200", {})
            if "value" in mine:
                line["engine_tok_per_s"] = mine
        print(json.dumps(line), flush=True)
    if not parity["ok"]:
        raise SystemExit("parity_check failed: the timed launch's output is outside the tolerance")


def secondary(dev, hbm_peak_gbs, only=None, compare=None):
    """Other kernels of the path, 1 GPU, device-timed (median of 20 after 3 warm-ups, L2
    flushed between iterations).  `compare`: also time the library kernels the reference calls on
    the same inputs (default: yes for the whole set, as asked for a single kernel)."""
    import torch
    from nano_vllm_b200 import attention as A, workloads as W

    if compare is None:
        compare = only is None
    tf_peak = measured_peaks().get("bf16_tflops")

    def med(fn, iters=20):
        for _ in range(3):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for a, b in evs:
            flush.zero_()  # evict L2 (126 MB) between iterations
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in evs)

    def tf_line(ms, fl):
        d = {"us": round(ms * 1e3, 1), "TFLOP/s": round(fl / ms / 1e9, 1)}
        if tf_peak:
            d["frac_of_bf16_peak"] = round(fl / ms / 1e9 / tf_peak, 3)
        return d

    def bw_line(ms, nb):
        return {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1), "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}

    fa = None
    if compare:
        try:
            import flash_attn as fa
        except Exception:
            fa = None
    res = {}
    if compare and fa is None and only in (None, "prefill", "prefill_long", "decode", "decode_long"):
        res["flash_attn"] = "unavailable: the flash_attn package does not import here"

    def decode_lines(name, case, iters=10, with_fa=True):
        B, Hq, Hkv, D = case.geometry
        nb = W.decode_bytes(case.context_lens.cpu(), Hq, Hkv, D)
        o = torch.empty_like(case.q)
        ms = med(lambda: A.decode_paged(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale, out=o), iters)
        res[name] = bw_line(ms, nb)
        torch.cuda.synchronize()
        res[name]["parity_check"] = parity_against_oracle(case, o, 4)
        if fa and with_fa:
            bt = case.block_tables.clamp(min=0)
            ms = med(lambda: fa.flash_attn_with_kvcache(case.q.unsqueeze(1), case.k_cache, case.v_cache,
                                                        cache_seqlens=case.context_lens, block_table=bt,
                                                        softmax_scale=case.scale, causal=True), iters)
            res["flash_attn_" + name] = bw_line(ms, nb)

    if only in (None, "store", "prefill"):
        pc = W.cfg2_prefill(dev)
        n = pc.k.shape[0]
        if only in (None, "store"):
            ms = med(lambda: A.store_kvcache(pc.k, pc.v, pc.k_cache, pc.v_cache, pc.slot_mapping))
            res["store_kvcache_cfg2"] = bw_line(ms, W.store_bytes(n, 8 * 128))
        if only in (None, "prefill"):
            A.store_kvcache(pc.k, pc.v, pc.k_cache, pc.v_cache, pc.slot_mapping)
            lq = (pc.cu_seqlens_q[1:] - pc.cu_seqlens_q[:-1]).tolist()
            lk = (pc.cu_seqlens_k[1:] - pc.cu_seqlens_k[:-1]).tolist()
            fl = W.prefill_flops(lq, lk, 16, 128)
            o = torch.empty_like(pc.q)
            ms = med(lambda: A.prefill_varlen(pc.q, pc.k_cache, pc.v_cache, pc.cu_seqlens_q, pc.cu_seqlens_k,
                                              pc.max_seqlen_q, pc.max_seqlen_k, pc.scale,
                                              block_tables=pc.block_tables, out=o))
            res["prefill_cfg2_paged"] = tf_line(ms, fl)
            if fa:
                bt = pc.block_tables.clamp(min=0)
                ms = med(lambda: fa.flash_attn_varlen_func(pc.q, pc.k_cache, pc.v_cache, max_seqlen_q=pc.max_seqlen_q,
                                                           cu_seqlens_q=pc.cu_seqlens_q, max_seqlen_k=pc.max_seqlen_k,
                                                           cu_seqlens_k=pc.cu_seqlens_k, softmax_scale=pc.scale,
                                                           causal=True, block_table=bt))
                res["flash_attn_prefill_cfg2_paged"] = tf_line(ms, fl)
            del o
        del pc
    if only in (None, "prefill_long"):
        # the engine's warm-up shape: 4 sequences of 4096 tokens, packed K/V, Qwen3-0.6B heads
        pl = W.make_prefill_case(9, 4, 1, 1, 16, 8, 128, device=dev, lengths=[4096] * 4, with_cache=False)
        fl = W.prefill_flops([4096] * 4, [4096] * 4, 16, 128)
        o = torch.empty_like(pl.q)
        ms = med(lambda: A.prefill_varlen(pl.q, pl.k, pl.v, pl.cu_seqlens_q, pl.cu_seqlens_k, 4096, 4096, pl.scale, out=o))
        res["prefill_4x4096_packed"] = tf_line(ms, fl)
        if fa and only is not None:
            ms = med(lambda: fa.flash_attn_varlen_func(pl.q, pl.k, pl.v, max_seqlen_q=4096, cu_seqlens_q=pl.cu_seqlens_q,
                                                       max_seqlen_k=4096, cu_seqlens_k=pl.cu_seqlens_k,
                                                       softmax_scale=pl.scale, causal=True))
            res["flash_attn_prefill_4x4096_packed"] = tf_line(ms, fl)
        del pl, o
    if only in (None, "prefill_d64"):
        # the prompt lengths of the prefill configuration in Qwen2-0.5B geometry (14 q / 2 kv heads, head_dim 64)
        pd = W.make_prefill_case(2, 64, 100, 1024, device=dev, **W.QWEN2_05B)
        A.store_kvcache(pd.k, pd.v, pd.k_cache, pd.v_cache, pd.slot_mapping)
        lq = (pd.cu_seqlens_q[1:] - pd.cu_seqlens_q[:-1]).tolist()
        lk = (pd.cu_seqlens_k[1:] - pd.cu_seqlens_k[:-1]).tolist()
        fl = W.prefill_flops(lq, lk, 14, 64)
        o = torch.empty_like(pd.q)
        ms = med(lambda: A.prefill_varlen(pd.q, pd.k_cache, pd.v_cache, pd.cu_seqlens_q, pd.cu_seqlens_k,
                                          pd.max_seqlen_q, pd.max_seqlen_k, pd.scale,
                                          block_tables=pd.block_tables, out=o))
        res["prefill_cfg2_lengths_qwen2_d64"] = tf_line(ms, fl)
        del pd, o
    if only in (None, "decode"):
        # the headline workload (batch 256, Qwen3-8B geometry), kernel only, next to the library kernel
        c4 = W.cfg4_decode(1, 0, dev)
        decode_lines("decode_cfg4_b256", c4)
        del c4
    if only == "decode_tp8":
        # one rank's shard of the headline workload under 8-way tensor parallelism (4 q / 1 kv head)
        c8 = W.cfg4_decode(8, 0, dev)
        decode_lines("decode_cfg4_b256_tp8_shard", c8, 20)
        del c8
    if only == "decode_engine":
        # what a decode step of the end-to-end workload looks like to one layer: Qwen3-0.6B heads, 256
        # sequences of 100-2048 tokens, table as wide as max_model_len = 4096 allows
        ce = W.make_decode_case(3, 256, 100, 2048, device=dev, table_width=16, **W.QWEN3_06B)
        decode_lines("decode_qwen3_0.6b_b256_ctx100-2048", ce, 20)
        del ce
    if only in (None, "sampler"):
        # the engine's decode-step tail: one token per row of [256, 151936] bf16 logits, T = 0.6
        lg = (torch.randn(256, 151936, device=dev) * 2).to(torch.bfloat16)
        tt = torch.full((256,), 0.6, device=dev)
        tok = torch.empty(256, dtype=torch.int64, device=dev)
        nb = lg.numel() * 2 + 256 * 12
        calls = [0]

        def draw():
            calls[0] += 1
            A.sample_tokens(lg, tt, seed=1, step=calls[0], out=tok)
        ms = med(draw)
        res["sampler_b256_v151936_t0.6"] = bw_line(ms, nb)
        stock = ROOT / "baseline" / "_ref" / "nanovllm" / "layers" / "sampler.py"
        if compare and only is not None and stock.is_file():  # nano-vllm's own sampler module (plain torch), loaded by file
            import importlib.util
            spec = importlib.util.spec_from_file_location("_stock_sampler", stock)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            stock_sampler = mod.Sampler()
            with torch.inference_mode():
                ms = med(lambda: stock_sampler(lg, tt))
            res["stock_sampler_b256_v151936_t0.6"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1)}
        del lg, tt, tok
    if only in (None, "decode_long"):
        # long-context configuration: Qwen2-0.5B geometry, 512 sequences of 32768 tokens (8.6 GB of K+V),
        # whole on one GPU and as one rank's shard under 2-way tensor parallelism (7 q / 1 kv head)
        c5 = W.cfg5_decode(1, dev, batch=512)
        decode_lines("decode_cfg5_b512_ctx32768", c5, with_fa=only is not None)
        del c5
        torch.cuda.empty_cache()
        c5 = W.cfg5_decode(2, dev, batch=512)
        decode_lines("decode_cfg5_b512_ctx32768_tp2_shard", c5, with_fa=False)
        del c5
    return res


# ---- end to end: the engine ----------------------------------------------------------------

def _clean_env():
    """The environment of a child that is not a rank of this launcher."""
    drop = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK",
            "ROLE_WORLD_SIZE", "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS", "TORCH_NCCL_ASYNC_ERROR_HANDLING")
    return {k: v for k, v in os.environ.items() if k not in drop and not k.startswith("TORCHELASTIC_")}


def _wait_for_free_gpus(seconds=30):
    """The other ranks of the kernel benchmark exit on their own; wait until no other compute
    process is left on the visible GPUs (asked of nvidia-smi, so that this process opens no context
    on the other ranks' devices)."""
    deadline = time.time() + seconds
    me = str(os.getpid())
    while time.time() < deadline:
        try:
            out = subprocess.run(["nvidia-smi", "--query-compute-apps=pid", "--format=csv,noheader"],
                                 capture_output=True, text=True, timeout=20).stdout.split()
        except Exception:
            time.sleep(5)
            return
        if all(pid == me for pid in out):
            return
        time.sleep(0.5)


def engine_once(attn, tp, model, timeout):
    try:
        proc = subprocess.run([sys.executable, "-m", "nano_vllm_b200.e2e", "--attn", attn, "--tp", str(tp), "--model", model],
                              cwd=str(ROOT), capture_output=True, text=True, timeout=timeout, env=_clean_env())
        for ln in reversed(proc.stdout.strip().splitlines()):
            if ln.startswith("{"):
                d = json.loads(ln)
                return {k: d[k] for k in ("value", "unit", "attn", "tp", "num_seqs", "output_tokens", "seconds",
                                          "device_status_word", "unavailable") if k in d}
        return {"unavailable": (proc.stderr or proc.stdout)[-300:]}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


def engine_runs(tp):
    """Output tok/s of the unmodified nano-vllm engine (installed under baseline/_ref) on its own
    benchmark workload (256 requests, prompt and output lengths U[100,1024], temperature 0.6,
    random-init weights) at tensor-parallel size `tp`: with this package plugged in (attention
    layer, fused pre-attention step, one-pass sampler, one-launch decode inputs; the peer-memory
    all-reduce too when tp > 1) and stock (Triton + flash-attn + NCCL), Qwen3-0.6B at every tp and
    Qwen3-8B geometry when tp > 1.  Child processes under a shared wall-clock budget; what does
    not fit is reported as skipped."""
    if not (ROOT / "baseline" / "_ref" / "nanovllm").is_dir():
        return {"unavailable": "no nano-vllm install under baseline/_ref"}
    if tp > 1:
        _wait_for_free_gpus()
    mine = "b200-full-ar" if tp > 1 else "b200-full"
    plan = [("qwen3-0.6b", "b200", mine), ("qwen3-0.6b", "reference", "reference")]
    if tp > 1:
        plan += [("qwen3-8b", "b200", mine), ("qwen3-8b", "reference", "reference")]
    t0, res = time.time(), {}
    for model, key, attn in plan:
        left = ENGINE_BUDGET_S - (time.time() - t0)
        if left < 100:
            res.setdefault(model, {})[key] = {"unavailable": "skipped: time budget of the benchmark run spent"}
            continue
        res.setdefault(model, {})[key] = engine_once(attn, tp, model, min(300, left))
    for model, d in res.items():
        if "value" in d.get("b200", {}) and "value" in d.get("reference", {}):
            d["ratio"] = round(d["b200"]["value"] / d["reference"]["value"], 3)
    return res


# ---- single kernels ------------------------------------------------------------------------

def run_allreduce(args):
    """Latency of the peer-memory all-reduce next to NCCL's on the sizes a decode step sums; run
    under torchrun, one process per GPU.  Each size is timed with CUDA events over back-to-back
    calls after a warm-up (max over ranks), eagerly and replayed from a CUDA graph (how the
    engine's decode step issues them).  Rank 0 prints one JSON line per size."""
    import torch
    import torch.distributed as dist
    from nano_vllm_b200 import _lib
    from nano_vllm_b200.allreduce import PeerAllReduce

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    build_once(local, dist.barrier)
    iters = args.steps

    def timed(fn, n, warm=10):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / n * 1e3], device="cuda")  # us per call
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def graphed(fn, calls=8):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            fn()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(calls):
                    fn()
        return g, calls

    ar = PeerAllReduce(rank, world, 8 << 20, wait_ms=20000)
    ar.force_protocol(args.ar_protocol)
    for rows, hidden in ((16, 1024), (64, 1024), (256, 1024), (128, 4096), (256, 4096), (512, 4096)):
        x = (torch.randn(rows, hidden, generator=torch.Generator().manual_seed(rank)) * 0.5).to(torch.bfloat16).cuda()
        y1, y2 = x.clone(), x.clone()
        ar.all_reduce(y1)
        dist.all_reduce(y2)
        torch.cuda.synchronize()
        scratch = x.clone()
        line = {"kernel": "allreduce", "bytes": x.numel() * 2, "shape": [rows, hidden], "world": world,
                "protocol": ar.protocol(x.numel() * 2), "max_abs_diff_vs_nccl": float((y1.float() - y2.float()).abs().max())}
        line["peer_us"] = round(timed(lambda: ar.all_reduce(scratch), iters), 2)
        line["nccl_us"] = round(timed(lambda: dist.all_reduce(scratch), iters), 2)
        scratch.copy_(x)
        g, calls = graphed(lambda: ar.all_reduce(scratch))
        line["peer_graph_us"] = round(timed(g.replay, iters // calls + 1) / calls, 2)
        scratch.copy_(x)
        g2, calls = graphed(lambda: dist.all_reduce(scratch))
        line["nccl_graph_us"] = round(timed(g2.replay, iters // calls + 1) / calls, 2)
        line["status"] = _lib.read_status()
        if rank == 0:
            print(json.dumps(line), flush=True)
        del g, g2
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


def run_gemm_allreduce(args):
    """The row-parallel projection and its sum as one launch (PeerAllReduce.linear_all_reduce) next
    to the pairs it replaces -- torch's F.linear followed by the peer-memory all-reduce, and by
    NCCL's -- on the o_proj / down_proj shapes of a decode step; run under torchrun, one process
    per GPU, every variant replayed from a CUDA graph, max over ranks.  Rank 0 prints one JSON line
    per shape."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from nano_vllm_b200 import _lib
    from nano_vllm_b200.allreduce import PeerAllReduce

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    build_once(local, dist.barrier)
    iters = args.steps

    def timed_graph(fn, calls=8):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            fn()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(calls):
                    fn()
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = iters // calls + 1
        a.record()
        for _ in range(n):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / (n * calls) * 1e3], device="cuda")  # us per call
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t), 2)

    ar = PeerAllReduce(rank, world, 8 << 20, wait_ms=20000)
    shapes = [(name, tokens, hidden, k_total // world)
              for name, hidden, k_total in (("qwen3-8b o_proj", 4096, 4096), ("qwen3-8b down_proj", 4096, 12288),
                                            ("qwen3-0.6b o_proj", 1024, 2048), ("qwen3-0.6b down_proj", 1024, 3072))
              for tokens in (16, 64, 256)]
    for name, m, n, k in shapes:
        g = torch.Generator().manual_seed(1 + rank)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(n, k, generator=g) * (k * world) ** -0.5).to(torch.bfloat16).cuda()
        if not ar.linear_fits(x, w):
            continue
        fused = ar.linear_all_reduce(x, w)
        pair = ar.all_reduce(F.linear(x, w))
        torch.cuda.synchronize()
        out = torch.empty_like(fused)
        line = {"kernel": "gemm_allreduce", "layer": name, "tokens": m, "n": n, "k_per_rank": k, "world": world,
                "max_abs_diff_vs_pair": float((fused.float() - pair.float()).abs().max()),
                "out_abs_max": float(pair.float().abs().max())}
        line["fused_us"] = timed_graph(lambda: ar.linear_all_reduce(x, w, out))
        line["linear_us"] = timed_graph(lambda: F.linear(x, w))
        line["linear_peer_us"] = timed_graph(lambda: ar.all_reduce(F.linear(x, w)))
        line["linear_nccl_us"] = timed_graph(lambda: dist.all_reduce(F.linear(x, w)))
        line["status"] = _lib.read_status()
        if rank == 0:
            print(json.dumps(line), flush=True)
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


def run_one_kernel(args):
    if args.kernel == "allreduce":
        return run_allreduce(args)
    if args.kernel == "gemm_allreduce":
        return run_gemm_allreduce(args)
    import torch
    from nano_vllm_b200 import build as _build
    _build.build()
    torch.cuda.set_device(0)
    peak, _ = hbm_peak()
    print(json.dumps({"kernel": args.kernel, **secondary(torch.device("cuda", 0), peak, only=args.kernel,
                                                          compare=args.with_flash_attn)}), flush=True)


def main():
    args = parse_args()
    if args.kernel:
        return run_one_kernel(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
