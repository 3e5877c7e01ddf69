// One-shot all-reduce (sum, bf16) over peer memory, for the row-parallel projections that follow
// the attention layer.
//
// nano-vllm sums the partial outputs of o_proj and down_proj across tensor-parallel ranks with
// dist.all_reduce (nanovllm/layers/linear.py:195-199): 2 x layers NCCL calls per decode step on a
// [batch, hidden] bf16 tensor of 0.5-2 MiB, i.e. latency-bound.  Here every rank owns one device
// allocation that all its peers map through CUDA IPC:
//
//     [ flags: kMaxBlocks x kMaxRanks u32 | call counts | staging 0 | staging 1 | cells 0 | cells 1 |
//       result 0 | result 1 | result cells 0 | result cells 1 ]
//
// Four protocols, chosen by size and world (the same choice on every rank).
//
// SMALL tensors (2 x bytes x world <= max_bytes): flagged cells, in the manner of NCCL's
// low-latency protocol.  A cell is 16 bytes: 8 bytes of data and the call count twice
// {d0, count, d1, count}, written with one 16-byte store; each 8-byte half validates itself, so a
// store that arrives in two halves is harmless.  Every thread pushes its cells straight into the
// cell area of every peer (region [buffer][source rank]), then polls its OWN area (local memory)
// until the cells of every peer carry this call's count, and sums in rank order.  No fence, no
// separate flag round trip, no block-wide barrier: one NVLink crossing of latency.
//
// MEDIUM tensors at more than two ranks: flagged cells in two shots.  Pushing every cell to every
// peer costs 2 x bytes x (world-1) on the wire; here the tensor is cut into `world` slices, a rank
// pushes the cells of slice j to its owner j only, the owner sums them as they arrive and pushes
// the cells of the result to every peer: 4 x bytes x (world-1)/world per rank, two NVLink
// crossings of latency, still no fence, no flag round trip and no block-wide barrier.
//
// LARGER tensors, one shot: staging + flags.
//
// One call = one kernel on every rank, same grid everywhere.  Block b of rank r
//   1. copies its slice of the input into r's staging buffer (e & 1), e = the block's call count,
//   2. publishes 2e into flag (b, r) of every peer (st.release.sys through the peer mapping),
//   3. waits until its own flags (b, p) have reached 2e for every peer p (ld.acquire.sys; bounded
//      by a clock limit, after which the status word gets NVLLM_STATUS_TIMEOUT, a latch in the
//      allocation makes later calls give up at once, and the block carries on without hanging),
//   4. sums slice b of every rank's staging buffer in rank order, in fp32, and writes bf16.
// Every rank adds the same numbers in the same order, so all ranks hold bit-identical results.
// Two staging buffers used in turn need no closing barrier: a peer cannot reach call e+2 (which
// overwrites buffer e & 1) before this rank has published e+1, which it does after reading.
//
// LARGER tensors at more than two ranks, two shots (reduce-scatter, then all-gather): one shot
// makes every rank pull world-1 whole tensors; here a rank moves 2 (world-1)/world of one.  The
// tensor is cut into `world` slices, slice j owned by rank j.  Block b of rank r
//   1. pushes its part of slice j of the input straight into rank j's staging buffer, region
//      [source r], for every peer j; publishes 2e-1 to flag (b, r) of every peer; waits for 2e-1,
//   2. sums its part of slice r (own input + the world-1 regions of its staging buffer) in rank
//      order in fp32, writes the bf16 result to `out` and pushes it into the result buffer (e & 1)
//      of every peer; publishes 2e; waits for 2e,
//   3. copies the other slices' results from its own result buffer to `out`.
// A slice is summed by exactly one rank, so all ranks hold the same bits.  The flag values of the
// two staging protocols interleave (2e-1 < 2e < 2(e+1)-1), so calls of either kind can follow
// each other, and the two-buffer argument above covers both areas.
// All accesses to peer memory are plain 16-byte loads and stores issued by each thread itself:
// no bulk-copy engine and no switch-side broadcast or reduction object is involved.  Flags and
// call counts live in device memory, so a captured graph replays correctly.
#include <cooperative_groups.h>

#include <cstring>

#include "allreduce.cuh"

namespace nvllm {
namespace ar {

struct Params {
  const uint4* in;
  uint4* out;
  int64_t n16;        // 16-byte vectors (8 bf16 each)
  int64_t tail_elems; // elements after the last whole vector (handled by block 0)
  int64_t stage_bytes;
  long long wait_cycles;  // a wait for a peer gives up after this many SM clocks
  int rank, world;
  int force;  // Protocol: kAuto, or the protocol to use (measurement aid; same on every rank)
  Peers peers;
  int* status;
};

// The work of block `b` (of `nblocks`) on behalf of rank `rank`.
__device__ void allreduce_block(const Params& p, int rank, int b, int nblocks) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  unsigned char* own = p.peers.base[rank];
  uint32_t* epochs = reinterpret_cast<uint32_t*>(own + kEpochOff);
  uint32_t* broken = reinterpret_cast<uint32_t*>(own + kBrokenOff);
  if (tid == 0) {
    s_epoch = epochs[b] + 1;
    s_abort = *reinterpret_cast<volatile uint32_t*>(broken) != 0;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  const int64_t stage_off = kHeaderBytes + static_cast<int64_t>(e & 1) * p.stage_bytes;
  const int64_t v0 = p.n16 * b / nblocks, v1 = p.n16 * (b + 1) / nblocks;
  const bool has_tail = b == 0 && p.tail_elems > 0;

  // 1. own slice -> own staging buffer
  uint4* stage = reinterpret_cast<uint4*>(own + stage_off);
  for (int64_t v = v0 + tid; v < v1; v += blockDim.x) stage[v] = p.in[v];
  if (has_tail && tid < p.tail_elems) {
    const __nv_bfloat16* in_t = reinterpret_cast<const __nv_bfloat16*>(p.in + p.n16);
    reinterpret_cast<__nv_bfloat16*>(stage + p.n16)[tid] = in_t[tid];
  }
  __threadfence_system();
  __syncthreads();

  // 2. publish, 3. wait (one thread per peer)
  if (tid < p.world && tid != rank) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(p.peers.base[tid]) + b * kMaxRanks + rank;
    st_release_sys(theirs, 2 * e);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(own) + b * kMaxRanks + tid;
    if (!s_abort) {
      const long long t0 = clock64();
      while (static_cast<int32_t>(ld_acquire_sys(mine) - 2 * e) < 0) {
        if (clock64() - t0 > p.wait_cycles) {
          atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
          *reinterpret_cast<volatile uint32_t*>(broken) = 1;  // later calls do not wait again
          break;
        }
      }
    }
  }
  __syncthreads();

  // 4. sum in rank order
  for (int64_t v = v0 + tid; v < v1; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      const uint4* src = reinterpret_cast<const uint4*>(p.peers.base[r] + stage_off);
      add8(acc, ld_volatile16(src + v));
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    p.out[v] = o;
  }
  if (has_tail && tid < p.tail_elems) {
    float acc = 0.f;
    for (int r = 0; r < p.world; ++r) {
      const volatile __nv_bfloat16_raw* src =
          reinterpret_cast<const volatile __nv_bfloat16_raw*>(p.peers.base[r] + stage_off + p.n16 * 16);
      __nv_bfloat16_raw raw;
      raw.x = src[tid].x;
      acc += __bfloat162float(__nv_bfloat16(raw));
    }
    reinterpret_cast<__nv_bfloat16*>(p.out + p.n16)[tid] = __float2bfloat16(acc);
  }
  if (tid == 0) epochs[b] = e;
}

// Cell protocol: the work of block `b` on behalf of rank `rank`.  n_cells = ceil(n_elems / 4).
__device__ void allreduce_cells_block(const Params& p, int rank, int b, int nblocks) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  unsigned char* own = p.peers.base[rank];
  uint32_t* epochs = reinterpret_cast<uint32_t*>(own + kCellEpochOff);
  uint32_t* broken = reinterpret_cast<uint32_t*>(own + kBrokenOff);
  if (tid == 0) {
    s_epoch = epochs[b] + 1;
    s_abort = *reinterpret_cast<volatile uint32_t*>(broken) != 0;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  const int64_t n_elems = p.n16 * 8 + p.tail_elems;
  const int64_t n_cells = (n_elems + 3) / 4;
  const int64_t cells_cap = p.stage_bytes / 16 / p.world;  // cells per source rank in one buffer
  const int64_t area_off = kHeaderBytes + 2 * p.stage_bytes + static_cast<int64_t>(e & 1) * p.stage_bytes;
  const int64_t c0 = n_cells * b / nblocks, c1 = n_cells * (b + 1) / nblocks;
  const uint2* in2 = reinterpret_cast<const uint2*>(p.in);
  uint2* out2 = reinterpret_cast<uint2*>(p.out);
  const __nv_bfloat16* in_e = reinterpret_cast<const __nv_bfloat16*>(p.in);
  __nv_bfloat16* out_e = reinterpret_cast<__nv_bfloat16*>(p.out);

  auto load_own = [&](int64_t c) {
    if (4 * c + 4 <= n_elems) return in2[c];
    __nv_bfloat16 t[4];  // the ragged last cell: missing elements are zero
    for (int k = 0; k < 4; ++k) t[k] = 4 * c + k < n_elems ? in_e[4 * c + k] : __float2bfloat16(0.f);
    return *reinterpret_cast<const uint2*>(t);
  };

  // push this rank's cells into every peer's area, region [source = rank]
  for (int64_t c = c0 + tid; c < c1; c += blockDim.x) {
    const uint2 d = load_own(c);
    const uint4 cell = make_uint4(d.x, e, d.y, e);
    for (int r = 0; r < p.world; ++r) {
      if (r == rank) continue;
      uint4* dst = reinterpret_cast<uint4*>(p.peers.base[r] + area_off) + rank * cells_cap + c;
      st_volatile16(dst, cell);
    }
  }
  // collect: own area, regions [source = r]; every source's cell is requested before the first is
  // looked at (one memory latency instead of world-1 in a row), then summed in rank order
  bool gave_up = s_abort;
  // a cell of this call (first try: the value already loaded), or after the clock limit whatever is there
  auto settle = [&](const uint4* src, uint4 v) {
    if (!gave_up && (v.y != e || v.w != e)) {
      const long long t0 = clock64();
      do {
        v = ld_volatile16(src);
        if (clock64() - t0 > p.wait_cycles) {
          atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
          *reinterpret_cast<volatile uint32_t*>(broken) = 1;
          gave_up = true;
          break;
        }
      } while (v.y != e || v.w != e);
    }
    return v;
  };
  for (int64_t c = c0 + tid; c < c1; c += blockDim.x) {
    const uint4* mine = reinterpret_cast<const uint4*>(own + area_off) + c;
    uint4 got[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < p.world && r != rank) got[r] = ld_volatile16(mine + r * cells_cap);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r >= p.world) continue;
      if (r == rank) {
        const uint2 d = load_own(c);
        add4(acc, d.x, d.y);
      } else {
        const uint4 v = settle(mine + r * cells_cap, got[r]);
        add4(acc, v.x, v.z);
      }
    }
    uint2 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    if (4 * c + 4 <= n_elems) {
      out2[c] = o;
    } else {
      const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(&o);
      for (int k = 0; k < 4; ++k)
        if (4 * c + k < n_elems) out_e[4 * c + k] = t[k];
    }
  }
  __syncthreads();
  if (tid == 0) epochs[b] = e;
}

// Flagged cells in two shots: the work of block `b` on behalf of rank `rank`.
__device__ void allreduce_cells_twoshot_block(const Params& p, int rank, int b, int nblocks) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  const int w = p.world;
  unsigned char* own = p.peers.base[rank];
  uint32_t* epochs = reinterpret_cast<uint32_t*>(own + kCellEpochOff);
  uint32_t* broken = reinterpret_cast<uint32_t*>(own + kBrokenOff);
  if (tid == 0) {
    s_epoch = epochs[b] + 1;
    s_abort = *reinterpret_cast<volatile uint32_t*>(broken) != 0;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  const int64_t n_elems = p.n16 * 8 + p.tail_elems;
  const int64_t n_cells = (n_elems + 3) / 4;
  const int64_t cells_cap = p.stage_bytes / 16 / w;  // cells per source rank in a first-shot area
  const int64_t area1 = kHeaderBytes + (2 + static_cast<int64_t>(e & 1)) * p.stage_bytes;  // [source][cell of my slice]
  const int64_t area2 = kHeaderBytes + (6 + static_cast<int64_t>(e & 1)) * p.stage_bytes;  // [cell of the tensor]
  const uint2* in2 = reinterpret_cast<const uint2*>(p.in);
  uint2* out2 = reinterpret_cast<uint2*>(p.out);
  const __nv_bfloat16* in_e = reinterpret_cast<const __nv_bfloat16*>(p.in);
  __nv_bfloat16* out_e = reinterpret_cast<__nv_bfloat16*>(p.out);
  auto load_own = [&](int64_t c) {
    if (4 * c + 4 <= n_elems) return in2[c];
    __nv_bfloat16 t[4];  // the ragged last cell: missing elements are zero
    for (int k = 0; k < 4; ++k) t[k] = 4 * c + k < n_elems ? in_e[4 * c + k] : __float2bfloat16(0.f);
    return *reinterpret_cast<const uint2*>(t);
  };
  auto store_out = [&](int64_t c, const uint2& o) {
    if (4 * c + 4 <= n_elems) {
      out2[c] = o;
    } else {
      const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(&o);
      for (int k = 0; k < 4; ++k)
        if (4 * c + k < n_elems) out_e[4 * c + k] = t[k];
    }
  };
  // this block's part [lo, hi) of slice j (slices and parts in cells); 32-bit arithmetic (at most
  // 2^22 cells x 8 ranks, a slice x 128 blocks): a 64-bit division costs ~100 cycles, and there
  // are four per slice and phase
  const uint32_t nc32 = static_cast<uint32_t>(n_cells), w32 = static_cast<uint32_t>(w), nb32 = static_cast<uint32_t>(nblocks);
  auto part = [&](int j, int64_t& s0, int64_t& lo, int64_t& hi) {
    const uint32_t a = nc32 * static_cast<uint32_t>(j) / w32;
    const uint32_t len = nc32 * static_cast<uint32_t>(j + 1) / w32 - a;
    s0 = a;
    lo = a + len * static_cast<uint32_t>(b) / nb32;
    hi = a + len * static_cast<uint32_t>(b + 1) / nb32;
  };
  bool gave_up = s_abort;
  // a cell of this call (first try: the value already loaded), or after the clock limit whatever is there
  auto settle = [&](const uint4* src, uint4 v) {
    if (!gave_up && (v.y != e || v.w != e)) {
      const long long t0 = clock64();
      do {
        v = ld_volatile16(src);
        if (clock64() - t0 > p.wait_cycles) {
          atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
          *reinterpret_cast<volatile uint32_t*>(broken) = 1;
          gave_up = true;
          break;
        }
      } while (v.y != e || v.w != e);
    }
    return v;
  };

  // 1. my cells of every other slice go to the slice's owner, region [source = rank]
  for (int k = 1; k < w; ++k) {
    const int j = (rank + k) % w;
    int64_t s0, lo, hi;
    part(j, s0, lo, hi);
    uint4* dst = reinterpret_cast<uint4*>(p.peers.base[j] + area1) + rank * cells_cap - s0;
    for (int64_t c = lo + tid; c < hi; c += blockDim.x) {
      const uint2 d = load_own(c);
      st_volatile16(dst + c, make_uint4(d.x, e, d.y, e));
    }
  }
  // 2. my slice: sum in rank order as the peers' cells arrive; result to `out` and to every peer
  {
    int64_t s0, lo, hi;
    part(rank, s0, lo, hi);
    const uint4* mine = reinterpret_cast<const uint4*>(own + area1);
    for (int64_t c = lo + tid; c < hi; c += blockDim.x) {
      // every source's cell is requested before the first is looked at
      uint4 got[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < w && r != rank) got[r] = ld_volatile16(mine + r * cells_cap + (c - s0));
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r >= w) continue;
        if (r == rank) {
          const uint2 d = load_own(c);
          add4(acc, d.x, d.y);
        } else {
          const uint4 v = settle(mine + r * cells_cap + (c - s0), got[r]);
          add4(acc, v.x, v.z);
        }
      }
      uint2 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      store_out(c, o);
      const uint4 cell = make_uint4(o.x, e, o.y, e);
      for (int k = 1; k < w; ++k) {
        const int j = (rank + k) % w;
        st_volatile16(reinterpret_cast<uint4*>(p.peers.base[j] + area2) + c, cell);
      }
    }
  }
  // 3. the other slices' results arrive in my result-cell area
  const uint4* results = reinterpret_cast<const uint4*>(own + area2);
  for (int k = 1; k < w; ++k) {
    const int j = (rank + k) % w;
    int64_t s0, lo, hi;
    part(j, s0, lo, hi);
    for (int64_t c = lo + tid; c < hi; c += 4 * blockDim.x) {  // four cells in flight per thread
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c + k * blockDim.x < hi) v[k] = ld_volatile16(results + c + k * blockDim.x);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (c + k * blockDim.x >= hi) continue;
        v[k] = settle(results + c + k * blockDim.x, v[k]);
        store_out(c + k * blockDim.x, make_uint2(v[k].x, v[k].z));
      }
    }
  }
  __syncthreads();
  if (tid == 0) epochs[b] = e;
}

// Two shots: the work of block `b` (of `nblocks`) on behalf of rank `rank`.  tail_elems == 0.
__device__ void allreduce_twoshot_block(const Params& p, int rank, int b, int nblocks) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  const int w = p.world;
  unsigned char* own = p.peers.base[rank];
  uint32_t* epochs = reinterpret_cast<uint32_t*>(own + kEpochOff);
  uint32_t* broken = reinterpret_cast<uint32_t*>(own + kBrokenOff);
  if (tid == 0) {
    s_epoch = epochs[b] + 1;
    s_abort = *reinterpret_cast<volatile uint32_t*>(broken) != 0;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  const int64_t stage_off = kHeaderBytes + static_cast<int64_t>(e & 1) * p.stage_bytes;
  const int64_t result_off = kHeaderBytes + (4 + static_cast<int64_t>(e & 1)) * p.stage_bytes;
  const int64_t slice_cap = p.stage_bytes / 16 / w;  // vectors per source region of a staging buffer
  // this block's part [lo, hi) of slice j
  auto part = [&](int j, int64_t& s0, int64_t& lo, int64_t& hi) {
    s0 = p.n16 * j / w;
    const int64_t len = p.n16 * (j + 1) / w - s0;
    lo = s0 + len * b / nblocks;
    hi = s0 + len * (b + 1) / nblocks;
  };
  // publish `value` to flag (b, rank) of every peer and wait for the peers' (one thread per peer)
  auto handshake = [&](uint32_t value) {
    __threadfence_system();
    __syncthreads();
    if (tid < w && tid != rank) {
      uint32_t* theirs = reinterpret_cast<uint32_t*>(p.peers.base[tid]) + b * kMaxRanks + rank;
      st_release_sys(theirs, value);
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(own) + b * kMaxRanks + tid;
      if (!s_abort) {
        const long long t0 = clock64();
        while (static_cast<int32_t>(ld_acquire_sys(mine) - value) < 0) {
          if (clock64() - t0 > p.wait_cycles) {
            atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
            *reinterpret_cast<volatile uint32_t*>(broken) = 1;  // later calls do not wait again
            break;
          }
        }
      }
    }
    __syncthreads();
  };

  // 1. scatter: my part of every other slice goes to its owner, region [source = rank]
  for (int k = 1; k < w; ++k) {
    const int j = (rank + k) % w;  // every rank starts with another peer
    int64_t s0, lo, hi;
    part(j, s0, lo, hi);
    uint4* dst = reinterpret_cast<uint4*>(p.peers.base[j] + stage_off) + rank * slice_cap - s0;
    for (int64_t v = lo + tid; v < hi; v += blockDim.x) dst[v] = p.in[v];
  }
  handshake(2 * e - 1);

  // 2. reduce my part of my own slice in rank order; result to `out` and to every peer
  {
    int64_t s0, lo, hi;
    part(rank, s0, lo, hi);
    const uint4* stage = reinterpret_cast<const uint4*>(own + stage_off);
    for (int64_t v = lo + tid; v < hi; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < w; ++r) add8(acc, r == rank ? p.in[v] : ld_volatile16(stage + r * slice_cap + (v - s0)));
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      p.out[v] = o;
      for (int k = 1; k < w; ++k) {
        const int j = (rank + k) % w;
        reinterpret_cast<uint4*>(p.peers.base[j] + result_off)[v] = o;
      }
    }
  }
  handshake(2 * e);

  // 3. gather: the other owners' results are in my result buffer
  const uint4* result = reinterpret_cast<const uint4*>(own + result_off);
  for (int k = 1; k < w; ++k) {
    const int j = (rank + k) % w;
    int64_t s0, lo, hi;
    part(j, s0, lo, hi);
    for (int64_t v = lo + tid; v < hi; v += blockDim.x) p.out[v] = ld_volatile16(result + v);
  }
  if (tid == 0) epochs[b] = e;
}

// Which protocol a call uses: a pure function of (size, world, buffer size, forced choice), so
// every rank picks the same.
__host__ __device__ inline int pick_protocol(int64_t n16, int64_t tail_elems, int64_t stage_bytes, int world, int force) {
  const int64_t n_elems = n16 * 8 + tail_elems;
  const bool cells_fit = 2 * ((n_elems + 3) / 4 * 8) * world <= stage_bytes;
  const bool twoshot_fits = world > 2 && tail_elems == 0 && (n16 + world - 1) / world <= stage_bytes / 16 / world;
  const int64_t n_cells = (n_elems + 3) / 4;
  const bool cells_twoshot_fits = world > 2 && (n_cells + world - 1) / world <= stage_bytes / 16 / world && n_cells * 16 <= stage_bytes &&
                                  n_cells <= (1 << 25);  // the slices are cut with 32-bit arithmetic
  if (force == kCells && cells_fit) return kCells;
  if (force == kCellsTwoShot && cells_twoshot_fits) return kCellsTwoShot;
  if (force == kTwoShot && twoshot_fits) return kTwoShot;
  if (force == kOneShot) return kOneShot;
  if (cells_fit && (world == 2 || n_elems * 2 <= kCellsOneShotMaxBytes)) return kCells;
  if (cells_twoshot_fits) return kCellsTwoShot;
  if (twoshot_fits) return kTwoShot;
  return kOneShot;
}

__device__ __forceinline__ void allreduce_dispatch(const Params& p, int rank, int b, int nblocks) {
  const int proto = pick_protocol(p.n16, p.tail_elems, p.stage_bytes, p.world, p.force);
  if (proto == kCells) allreduce_cells_block(p, rank, b, nblocks);
  else if (proto == kCellsTwoShot) allreduce_cells_twoshot_block(p, rank, b, nblocks);
  else if (proto == kTwoShot) allreduce_twoshot_block(p, rank, b, nblocks);
  else allreduce_block(p, rank, b, nblocks);
}

__global__ void __launch_bounds__(kThreads) allreduce_kernel(const Params p) {
  allreduce_dispatch(p, p.rank, blockIdx.x, gridDim.x);
}

// All ranks in ONE launch on one device (blockIdx.y = rank; in/out per rank): the only legal way
// to run the hand-shake with fewer GPUs than ranks, since blocks that wait on each other must be
// resident together (cooperative launch).
struct EmuParams {
  Params base;
  const uint4* in[kMaxRanks];
  uint4* out[kMaxRanks];
  int absent_rank;  // this rank's blocks leave at once (a peer that never arrives); -1 = none
};
__global__ void __launch_bounds__(kThreads) allreduce_emulated_kernel(const EmuParams ep) {
  Params p = ep.base;
  const int rank = blockIdx.y;
  if (rank == ep.absent_rank) return;
  p.in = ep.in[rank];
  p.out = ep.out[rank];
  allreduce_dispatch(p, rank, blockIdx.x, gridDim.x);
}

// ---- host state (one per device of this process): declared in allreduce.cuh -----------------
static State g_state[64];

State* current_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return &g_state[dev];
}


}  // namespace ar
}  // namespace nvllm

using namespace nvllm;

extern "C" int64_t nvllm_ar_handle_bytes(void) { return static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)); }

extern "C" int nvllm_ar_init(int32_t rank, int32_t world, int64_t max_bytes, void* handle_out) {
  ar::State* s = ar::current_state();
  if (!s) return fail(NVLLM_E_NO_DEVICE, "ar_init: no CUDA device is usable");
  if (s->ready) return fail(NVLLM_E_GEOMETRY, "ar_init: already initialised on this device (call nvllm_ar_shutdown first)");
  if (world < 2 || world > ar::kMaxRanks || rank < 0 || rank >= world)
    return fail(NVLLM_E_GEOMETRY, "ar_init: rank=%d world=%d invalid (2..%d ranks)", rank, world, ar::kMaxRanks);
  if (max_bytes <= 0 || max_bytes % 16) return fail(NVLLM_E_GEOMETRY, "ar_init: max_bytes must be a positive multiple of 16");
  if (!handle_out) return fail(NVLLM_E_NULL, "ar_init: NULL handle_out");
  const size_t total = static_cast<size_t>(ar::kHeaderBytes + ar::kAreas * max_bytes);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, total);
  if (e == cudaSuccess) e = cudaMemset(p, 0, total);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (p) cudaFree(p);
    return fail(NVLLM_E_CUDA, "ar_init: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle_out, &h, sizeof(h));
  s->ready = true;
  s->connected = false;
  s->rank = rank;
  s->world = world;
  s->stage_bytes = max_bytes;
  s->own = static_cast<unsigned char*>(p);
  for (int r = 0; r < ar::kMaxRanks; ++r) s->peers.base[r] = nullptr;
  s->peers.base[rank] = s->own;
  return NVLLM_OK;
}

extern "C" int nvllm_ar_connect(const void* all_handles) {
  ar::State* s = ar::current_state();
  if (!s || !s->ready) return fail(NVLLM_E_GEOMETRY, "ar_connect: nvllm_ar_init has not run on this device");
  if (!all_handles) return fail(NVLLM_E_NULL, "ar_connect: NULL handles");
  if (s->connected) return NVLLM_OK;
  const unsigned char* hs = static_cast<const unsigned char*>(all_handles);
  for (int r = 0; r < s->world; ++r) {
    if (r == s->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, hs + static_cast<size_t>(r) * sizeof(h), sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(NVLLM_E_CUDA, "ar_connect: cannot map rank %d's buffer: %s", r, cudaGetErrorString(e));
    }
    s->peers.base[r] = static_cast<unsigned char*>(p);
  }
  s->connected = true;
  return NVLLM_OK;
}

extern "C" int nvllm_ar_shutdown(void) {
  ar::State* s = ar::current_state();
  if (!s || !s->ready) return NVLLM_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < s->world; ++r)
    if (r != s->rank && s->peers.base[r]) cudaIpcCloseMemHandle(s->peers.base[r]);
  cudaFree(s->own);
  (void)cudaGetLastError();
  *s = ar::State{};
  return NVLLM_OK;
}

extern "C" int nvllm_ar_set_wait_ms(int64_t ms) {
  ar::State* s = ar::current_state();
  if (!s || !s->ready) return fail(NVLLM_E_GEOMETRY, "ar_set_wait_ms: nvllm_ar_init has not run on this device");
  if (ms < 1 || ms > 600000) return fail(NVLLM_E_GEOMETRY, "ar_set_wait_ms: %lld ms outside 1..600000", (long long)ms);
  s->wait_cycles = ms * 2000000ll;  // SM clocks at ~2 GHz
  return NVLLM_OK;
}

extern "C" int nvllm_ar_set_protocol(int32_t protocol) {
  ar::State* s = ar::current_state();
  if (!s || !s->ready) return fail(NVLLM_E_GEOMETRY, "ar_set_protocol: nvllm_ar_init has not run on this device");
  if (protocol < ar::kAuto || protocol > ar::kCellsTwoShot) return fail(NVLLM_E_GEOMETRY, "ar_set_protocol: %d is not 0..4", protocol);
  s->force = protocol;
  return NVLLM_OK;
}

extern "C" int nvllm_ar_protocol(int64_t n_elems, int32_t world, int64_t max_bytes, int32_t forced) {
  if (n_elems <= 0 || world < 2 || world > ar::kMaxRanks || max_bytes <= 0)
    return fail(NVLLM_E_GEOMETRY, "ar_protocol: sizes invalid");
  return ar::pick_protocol(n_elems / 8, n_elems % 8, max_bytes, world, forced);
}

extern "C" int64_t nvllm_ar_max_bytes(void) {
  ar::State* s = ar::current_state();
  return (s && s->connected) ? s->stage_bytes : 0;
}

extern "C" int nvllm_ar_allreduce(const void* in, void* out, int64_t n_elems, void* stream) {
  ar::State* s = ar::current_state();
  if (!s || !s->connected) return fail(NVLLM_E_GEOMETRY, "ar_allreduce: not connected (nvllm_ar_init + nvllm_ar_connect first)");
  if (n_elems < 0) return fail(NVLLM_E_GEOMETRY, "ar_allreduce: negative size");
  if (n_elems == 0) return NVLLM_OK;
  if (!in || !out) return fail(NVLLM_E_NULL, "ar_allreduce: NULL pointer argument");
  if (!aligned16(in) || !aligned16(out)) return fail(NVLLM_E_ALIGN, "ar_allreduce: in/out must be 16-byte aligned");
  if ((n_elems * 2 + 15) / 16 * 16 > s->stage_bytes)
    return fail(NVLLM_E_WORKSPACE, "ar_allreduce: %lld bytes exceed the %lld-byte staging buffers", (long long)(n_elems * 2),
                (long long)s->stage_bytes);
  ar::Params p;
  p.in = static_cast<const uint4*>(in);
  p.out = static_cast<uint4*>(out);
  p.n16 = n_elems / 8;
  p.tail_elems = n_elems % 8;
  p.stage_bytes = s->stage_bytes;
  p.wait_cycles = s->wait_cycles;
  p.rank = s->rank;
  p.world = s->world;
  p.force = s->force;
  p.peers = s->peers;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "ar_allreduce: no CUDA device is usable");
  ar::allreduce_kernel<<<ar::kGrid, ar::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launch();
  return check_launch("ar_allreduce launch");
}

extern "C" int64_t nvllm_ar_emulated_scratch_bytes(int32_t world, int64_t max_bytes) {
  return static_cast<int64_t>(world) * (ar::kHeaderBytes + ar::kAreas * max_bytes);
}

extern "C" int nvllm_ar_allreduce_emulated(int32_t world, const void* const* inputs, void* const* outputs, int64_t n_elems,
                                           void* scratch, int64_t scratch_bytes, int64_t max_bytes, int32_t absent_rank,
                                           int32_t protocol, void* stream) {
  if (world < 2 || world > ar::kMaxRanks) return fail(NVLLM_E_GEOMETRY, "ar_allreduce_emulated: world=%d invalid", world);
  if (protocol < ar::kAuto || protocol > ar::kCellsTwoShot) return fail(NVLLM_E_GEOMETRY, "ar_allreduce_emulated: protocol=%d invalid", protocol);
  if (!inputs || !outputs || !scratch) return fail(NVLLM_E_NULL, "ar_allreduce_emulated: NULL pointer argument");
  if (max_bytes <= 0 || max_bytes % 16 || n_elems <= 0 || (n_elems * 2 + 15) / 16 * 16 > max_bytes)
    return fail(NVLLM_E_GEOMETRY, "ar_allreduce_emulated: sizes invalid");
  if (scratch_bytes < nvllm_ar_emulated_scratch_bytes(world, max_bytes) || !aligned16(scratch))
    return fail(NVLLM_E_WORKSPACE, "ar_allreduce_emulated: scratch too small or misaligned");
  ar::EmuParams ep;
  ep.base.n16 = n_elems / 8;
  ep.base.tail_elems = n_elems % 8;
  ep.base.stage_bytes = max_bytes;
  ep.base.wait_cycles = sm100::kWaitLimitCycles;
  ep.base.rank = 0;
  ep.base.world = world;
  ep.base.force = protocol;
  ep.base.status = status_word();
  ep.base.in = nullptr;
  ep.base.out = nullptr;
  ep.absent_rank = absent_rank;
  if (!ep.base.status) return fail(NVLLM_E_NO_DEVICE, "ar_allreduce_emulated: no CUDA device is usable");
  for (int r = 0; r < ar::kMaxRanks; ++r) {
    ep.base.peers.base[r] = r < world ? static_cast<unsigned char*>(scratch) + r * (ar::kHeaderBytes + ar::kAreas * max_bytes) : nullptr;
    ep.in[r] = r < world ? static_cast<const uint4*>(inputs[r]) : nullptr;
    ep.out[r] = r < world ? static_cast<uint4*>(outputs[r]) : nullptr;
    if (r < world && (!aligned16(inputs[r]) || !aligned16(outputs[r])))
      return fail(NVLLM_E_ALIGN, "ar_allreduce_emulated: in/out must be 16-byte aligned");
  }
  // few blocks per rank so that world x blocks fit on the device at once; cooperative launch
  // refuses to start otherwise, instead of letting waiting blocks starve the ones they wait for
  void* args[] = {&ep};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ar::allreduce_emulated_kernel), dim3(ar::kEmulatedGrid, world),
                                              dim3(ar::kThreads), args, 0, static_cast<cudaStream_t>(stream));
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_CUDA, "ar_allreduce_emulated launch: %s", cudaGetErrorString(e));
  }
  return NVLLM_OK;
}
