"""Benchmark of the paged-attention path: paged GQA decode attention, HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 4): one decode step of one layer in Qwen3-8B geometry (32 query /
8 KV heads, head_dim 128), 256 sequences with context lengths uniform in [2048, 8192], KV
cache in 256-token blocks addressed through a scattered block table.  With N GPUs the heads
and the cache are sharded N ways (tensor parallelism: 32/N query and 8/N KV heads per rank,
identical lengths and tables on every rank); the path has no collective, so ranks only meet
at the timing barrier.  Total work is fixed as N grows ("strong" scaling).

A step = what the attention layer does for that batch: store_kvcache of the new token's K/V,
then paged decode (split-KV partial kernel + combine kernel).  `value` counts the step's
algorithmic bytes (every live K/V byte once, q, o, lengths, table entries, the stored rows)
over the device time of K steps with everything resident in HBM; `e2e` is the same step
driven from pinned host buffers (q, new K/V rows and metadata copied in, output copied out,
all inside the timed region).  The KV cache itself is the path's device-resident state in the
engine (it never lives on the host), so it is not part of the per-step host traffic.

`--impl reference` times the CPU restatement of the reference path (fp32 torch SDPA over
blocks gathered through the table, oracle/paged_attention_ref.py) on the host cores, on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
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
# DRAM bytes per algorithmic byte of the decode kernel, from the ncu capture summarised in
# profiles/decode_paged_kernel_qwen3-8b_batch32.md (dram__bytes_read.sum + dram__bytes_write.sum over
# the case's algorithmic bytes; traffic grows in proportion to the KV bytes read).
DECODE_TRAFFIC_PER_ALGO_BYTE = 1.008
CPU_SAMPLE_SEQS = 32        # sequences per step of the reference arm
CPU_BASELINE_SEQS = 128     # sequences in the cpu_baseline leg of our arm (10 passes)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="sequences in the decode batch")
    ap.add_argument("--no-secondary", action="store_true", help="skip the store/prefill/long-context extras")
    ap.add_argument("--no-engine", action="store_true",
                    help="skip the end-to-end nano-vllm engine run (output tok/s) that follows at 1 GPU")
    ap.add_argument("--kernel", default=None, choices=["prefill", "prefill_long", "prefill_d64", "store", "decode", "decode_long", "sampler"],
                    help="time only this secondary kernel on one GPU and print its line (profiling aid)")
    ap.add_argument("--with-flash-attn", action="store_true",
                    help="with --kernel: also time the library kernels the reference calls (flash-attn, Triton "
                         "store) on the same inputs, if they are importable")
    return ap.parse_args()


def workload_name(n):
    return (f"cfg4: Qwen3-8B geometry single-layer paged decode, batch 256, ctx U[2048,8192], block 256, "
            f"TP={n} ({32 // n}q/{8 // n}kv heads per rank, D=128)")


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (MEASURED_PEAKS.json absent)"


# ---- clocks --------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the
    timed region runs; falls back to one nvidia-smi query if NVML is not importable."""

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

def cpu_sample(case, n_seqs):
    """Compacts the first n_seqs sequences of a (device) decode case into a small host case:
    only their blocks are kept, renumbered, so the host copy stays small."""
    import torch
    from nano_vllm_b200 import workloads as W
    lens = case.context_lens[:n_seqs].cpu()
    bt = case.block_tables[:n_seqs].cpu()
    used = bt[bt >= 0].to(torch.int64)
    remap = torch.full((int(case.k_cache.shape[0]),), -1, dtype=torch.int32)
    remap[used] = torch.arange(used.numel(), dtype=torch.int32)
    new_bt = torch.where(bt >= 0, remap[bt.clamp(min=0).to(torch.int64)], torch.full_like(bt, -1))
    idx = used.to(case.k_cache.device)
    return W.DecodeCase(case.q[:n_seqs].cpu(), case.k_new[:n_seqs].cpu(), case.v_new[:n_seqs].cpu(),
                        case.k_cache[idx].cpu(), case.v_cache[idx].cpu(), lens, new_bt,
                        torch.zeros(n_seqs, dtype=torch.int32), case.scale)


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

def run_ours(args):
    import torch
    import torch.distributed as dist
    from nano_vllm_b200 import _lib, attention as A, build as _build, workloads as W

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
    _build.build()
    _lib.load()

    case = W.cfg4_decode(world, rank, dev, batch=args.batch)
    B, Hq, Hkv, D = case.geometry
    lens_host = case.context_lens.cpu()
    step_bytes_rank = W.decode_bytes(lens_host, Hq, Hkv, D) + W.store_bytes(B, Hkv * D)
    decode_bytes_rank = W.decode_bytes(lens_host, Hq, Hkv, D)
    out = torch.empty_like(case.q)
    stream = torch.cuda.current_stream()

    def step(ev=None):
        A.store_kvcache(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping)
        if ev:
            ev[0].record(stream)
        A.decode_paged(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale, out=out)
        if ev:
            ev[1].record(stream)

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

    # ---- device-resident timing
    for _ in range(max(args.warmup, 3)):
        step()
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    barrier()
    launches0 = _lib.launch_count()
    sampler.start()
    t_start.record(stream)
    for i in range(args.steps):
        step(kev[i])
    t_end.record(stream)
    barrier()
    clocks = sampler.stop()
    launches = _lib.launch_count() - launches0
    total_ms = max_over_ranks(t_start.elapsed_time(t_end))
    ms_per_step = total_ms / args.steps
    decode_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in kev) / args.steps)
    status = _lib.read_status()

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
        A.store_kvcache(devbuf["k_new"], devbuf["v_new"], case.k_cache, case.v_cache, devbuf["slot_mapping"])
        A.decode_paged(devbuf["q"], case.k_cache, case.v_cache, devbuf["context_lens"], devbuf["block_tables"], case.scale, out=out)
        out_host.copy_(out, non_blocking=True)
        stream.synchronize()  # the caller reads the result on the host

    for _ in range(3):
        e2e_step()
    barrier()
    w0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - w0) * 1e3) / args.steps

    total_bytes = step_bytes_rank * world  # same lengths on every rank, heads split evenly
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9
    peak, peak_src = hbm_peak()
    achieved = decode_bytes_rank / (decode_ms * 1e-3) / 1e9
    traffic = None if DECODE_TRAFFIC_PER_ALGO_BYTE is None else int(decode_bytes_rank * DECODE_TRAFFIC_PER_ALGO_BYTE)
    chunk, splits = _lib.decode_plan(B, case.block_tables.shape[1], Hq, Hkv, D)

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(world), "global_batch": B, "kv_bytes_per_step": int(total_bytes),
                   "split_kv": {"chunk_tokens": chunk, "max_splits": splits},
                   "l2": "inputs (KV cache shard) larger than L2, re-read every step; no flush needed",
                   "parallelism": f"tp{world}"},
        "pct_of_nominal_8TBps_per_gpu": round(100 * value / world / NOMINAL_HBM_GBS, 1),
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d * world), "d2h_bytes_per_step": int(d2h * world)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "decode_paged_kernel (+ decode_combine_kernel)", "achieved": round(achieved, 1),
                     "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4), "peak_source": peak_src,
                     "traffic": traffic, "algorithmic_bytes_per_launch": int(decode_bytes_rank),
                     "avg_launch_ms": round(decode_ms, 4)},
        "device_status_word": status,
    }

    if rank == 0 and world == 1:
        n_cpu = min(B, CPU_BASELINE_SEQS)
        sample_case = cpu_sample(case, n_cpu)
        gbs, dt, nbytes, threads = time_cpu_reference(sample_case, steps=10, warmup=1)
        line["cpu_baseline"] = {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"first {n_cpu} of {B} sequences, 10 timed passes of {dt * 1e3:.0f} ms "
                                          f"({nbytes / 1e6:.0f} MB algorithmic each)"}
        if not args.no_secondary:
            del sample_case
            line["secondary"] = secondary(dev, peak)
        if not args.no_engine and not args.no_secondary:
            del case, out
            torch.cuda.empty_cache()
            line["engine_tok_per_s"] = engine_run()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def secondary(dev, hbm_peak_gbs, only=None, compare=False):
    """Other kernels of the path, 1 GPU, device-timed (median of 20 after 3 warm-ups, L2
    flushed between iterations)."""
    import torch
    from nano_vllm_b200 import attention as A, workloads as W

    tf_peak = None
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            tf_peak = float(json.loads(p.read_text())["bf16_tflops"])
        except Exception:
            pass

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

    fa = None
    if compare:
        try:
            import flash_attn as fa
        except Exception:
            fa = None
    res = {}
    if only in (None, "store", "prefill"):
        pc = W.cfg2_prefill(dev)
        n = pc.k.shape[0]
        if only in (None, "store"):
            ms = med(lambda: A.store_kvcache(pc.k, pc.v, pc.k_cache, pc.v_cache, pc.slot_mapping))
            sb = W.store_bytes(n, 8 * 128)
            res["store_kvcache_cfg2"] = {"us": round(ms * 1e3, 1), "GB/s": round(sb / ms / 1e6, 1),
                                         "frac_of_hbm_peak": round(sb / ms / 1e6 / hbm_peak_gbs, 3)}
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
        if fa:
            ms = med(lambda: fa.flash_attn_varlen_func(pl.q, pl.k, pl.v, max_seqlen_q=4096, cu_seqlens_q=pl.cu_seqlens_q,
                                                       max_seqlen_k=4096, cu_seqlens_k=pl.cu_seqlens_k,
                                                       softmax_scale=pl.scale, causal=True))
            res["flash_attn_prefill_4x4096_packed"] = tf_line(ms, fl)
        del pl, o
    if only in (None, "prefill_d64"):
        # config-2 lengths in Qwen2-0.5B geometry (14 q / 2 kv heads, head_dim 64)
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
    if only == "decode":
        # the headline workload (config 4, batch 256), kernel only, next to the library kernel
        c4 = W.cfg4_decode(1, 0, dev)
        B, Hq, Hkv, D = c4.geometry
        nb = W.decode_bytes(c4.context_lens.cpu(), Hq, Hkv, D)
        o = torch.empty_like(c4.q)
        ms = med(lambda: A.decode_paged(c4.q, c4.k_cache, c4.v_cache, c4.context_lens, c4.block_tables, c4.scale, out=o), 10)
        res["decode_cfg4_b256"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1),
                                   "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}
        if fa:
            bt = c4.block_tables.clamp(min=0)
            ms = med(lambda: fa.flash_attn_with_kvcache(c4.q.unsqueeze(1), c4.k_cache, c4.v_cache,
                                                        cache_seqlens=c4.context_lens, block_table=bt,
                                                        softmax_scale=c4.scale, causal=True), 10)
            res["flash_attn_decode_cfg4_b256"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1),
                                                  "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}
        del c4, o
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
        res["sampler_b256_v151936_t0.6"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1),
                                            "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}
        stock = ROOT / "baseline" / "_ref" / "nanovllm" / "layers" / "sampler.py"
        if compare and stock.is_file():  # nano-vllm's own sampler module (plain torch), loaded by file
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
        c5 = W.cfg5_decode(1, dev, batch=256)
        B, Hq, Hkv, D = c5.geometry
        nb = W.decode_bytes(c5.context_lens.cpu(), Hq, Hkv, D)
        o = torch.empty_like(c5.q)
        ms = med(lambda: A.decode_paged(c5.q, c5.k_cache, c5.v_cache, c5.context_lens, c5.block_tables, c5.scale, out=o), 10)
        res["decode_cfg5_b256_ctx32768"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1),
                                            "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}
        if fa:
            bt = c5.block_tables.clamp(min=0)
            ms = med(lambda: fa.flash_attn_with_kvcache(c5.q.unsqueeze(1), c5.k_cache, c5.v_cache,
                                                        cache_seqlens=c5.context_lens, block_table=bt,
                                                        softmax_scale=c5.scale, causal=True), 10)
            res["flash_attn_decode_cfg5_b256_ctx32768"] = {"us": round(ms * 1e3, 1), "GB/s": round(nb / ms / 1e6, 1),
                                                           "frac_of_hbm_peak": round(nb / ms / 1e6 / hbm_peak_gbs, 3)}
    return res


def engine_run():
    """Output tok/s of the unmodified nano-vllm engine (installed under baseline/_ref) with the
    B200 attention layer, the fused pre-attention step and the one-pass sampler swapped in: the
    reference's own benchmark workload on random-init
    Qwen3-0.6B, 1 GPU (python -m nano_vllm_b200.e2e).  Runs as a child process with a time limit;
    any failure is reported as a string instead of a number."""
    if not (ROOT / "baseline" / "_ref" / "nanovllm").is_dir():
        return {"unavailable": "no nano-vllm install under baseline/_ref"}
    try:
        proc = subprocess.run([sys.executable, "-m", "nano_vllm_b200.e2e", "--attn", "b200-full"], cwd=str(ROOT),
                              capture_output=True, text=True, timeout=420)
        for ln in reversed(proc.stdout.strip().splitlines()):
            if ln.startswith("{"):
                d = json.loads(ln)
                return {k: d[k] for k in ("value", "unit", "model", "num_seqs", "output_tokens", "seconds", "attn") if k in d}
        return {"unavailable": (proc.stderr or proc.stdout)[-300:]}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


def run_one_kernel(args):
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
