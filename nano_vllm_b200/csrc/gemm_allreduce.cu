// Row-parallel projection and its all-reduce as ONE kernel: Y = sum over ranks of X_r W_r^T.
//
// nano-vllm's RowParallelLinear (nanovllm/layers/linear.py:176-199) computes F.linear on every
// tensor-parallel rank and sums the partial outputs with dist.all_reduce: two launches and a pass
// of the [tokens, hidden] partial through HBM.  Here the product runs on the tcgen05 tensor cores
// (operands by TMA tile loads into a ring of shared-memory stages, accumulator in TMEM) and the
// epilogue that reads the accumulator IS the all-reduce, in the flagged-cell protocols of
// allreduce.cu, tile by tile.  Two shots:
//
//   * the output is cut into tiles of 128 rows x bn columns (bn = 32, 64 or 128, the smallest
//     that leaves at most one tile per thread block), a tile into groups of 4 columns (one cell per
//     row); group c of tile t is owned by rank (t + c) mod world, so every block of every rank
//     pushes, sums and collects the same amount;
//   * every rank rounds its fp32 partial of a tile to bf16 (what F.linear would have returned);
//     the cells {d0, call count, d1, call count} of the groups it does not own go straight from
//     registers into the owner's cell area, region [tile][source rank][owner's k-th group];
//   * the owner adds the partials of its groups in rank order in fp32 as the cells arrive (all
//     sources' cells in flight at once), rounds once, writes its own output and pushes the result
//     cells into every peer's result-cell area;
//   * the other ranks copy those groups from their result-cell area to their output.
// At two ranks, and for small outputs at more (the rule of the plain all-reduce), one shot instead:
// every rank pushes its partial of every tile to every peer and sums for itself, one NVLink
// crossing.  A cell of a tile lives at (column group * 128 + row) * 16 bytes, so the 32 lanes of
// a warp (32 consecutive accumulator rows) write 512 contiguous bytes per store instruction.
//
// The kernel uses the same grid, the same per-block call counts and the same two alternating cell
// areas as the cell protocols of the plain all-reduce, so calls of either kind may follow each
// other in any order (the same order on every rank).  All waits are bounded: on expiry the status
// word gets NVLLM_STATUS_TIMEOUT, the latch in the rank's area makes later calls give up at once,
// and the block frees its tensor memory and ends normally.  Peer memory is only touched by plain
// 16-byte stores issued by each thread; TMA loads read this rank's own X and W.
#include <cooperative_groups.h>

#include <cstdlib>

#include "allreduce.cuh"
#include "prefill_tc.cuh"

namespace nvllm {
namespace gar {
using namespace sm100;
using namespace ar;

constexpr int BM = 128, BK = 64, NTHREADS = 192;
// Shared memory: [control 1 KB | ring | 16 KB that only the products' unused rows reach].  A stage
// holds a_rows x 64 elements of X and bn x 64 of W as 128-byte-swizzled rows; a_rows is the batch
// rounded up to 16 (128 when there are several row tiles).  The product always reads 128 rows of
// X from the stage's start: for a small batch the rows past a_rows are whatever follows in the
// ring (the W tile, later stages).  An output row depends on its own X row only, so that garbage
// ends in accumulator rows nobody reads, and a small batch's stages hold far more of k.  A stage
// covers ksub = 4, 2 or 1 k-blocks of 64 elements (one barrier round trip and one commit per
// stage: with one k-block per stage the issuing threads, not the memory system, set the pace).
constexpr int MAX_NST = 24;
constexpr int CTRL_BYTES = 1024, RING_BYTES = 192 * 1024, SLACK_BYTES = BM * 128;
constexpr int SMEM = CTRL_BYTES + RING_BYTES + SLACK_BYTES + 1024;  // + alignment slack
enum Bar { FULL0 = 0, EMPTY0 = MAX_NST, ACC_FULL = 2 * MAX_NST, ACC_FREE, DRAIN, NUM_BARS };
static_assert(NUM_BARS * 8 <= 512, "barrier area");

struct Maps {
  CUtensorMap x[kMaxRanks];  // [m, k] activations of each rank (one entry unless emulated)
  CUtensorMap w[kMaxRanks];  // [n, k] weight shard of each rank
};

struct Params {
  __nv_bfloat16* out[kMaxRanks];
  int64_t out_stride;  // elements between output rows
  int m, n, k, bn;
  int a_rows;          // rows of X per stage (box height of the X tensor map)
  int ksub;            // 64-element k-blocks per stage (one barrier round trip and one commit per stage)
  int nst;             // stages in the ring
  int one_shot;        // every rank sums every tile itself (one NVLink crossing) instead of the tile's owner
  int rank;            // >= 0: this process's rank; < 0: emulated, rank = blockIdx.x / nblocks
  int world, nblocks;  // thread blocks per rank
  int64_t stage_bytes;
  long long wait_cycles;
  Peers peers;
  int* status;
};

__global__ void __launch_bounds__(NTHREADS, 1) gemm_allreduce_kernel(const __grid_constant__ Maps maps, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = p.rank >= 0 ? p.rank : static_cast<int>(blockIdx.x) / p.nblocks;
  const int b = p.rank >= 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) % p.nblocks;
  const int mi = p.rank >= 0 ? 0 : rank;  // which tensor maps
  const int w = p.world, bn = p.bn;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + 520);
  volatile uint32_t* s_epoch = reinterpret_cast<volatile uint32_t*>(base_ptr + 524);
  volatile int* s_broken = reinterpret_cast<volatile int*>(base_ptr + 528);
  const uint32_t ring = base + CTRL_BYTES;
  // a stage = ksub sub-tiles of 64 k-elements, each [X rows | W rows] x 128 B
  const int NST = p.nst, ksub = p.ksub, a_bytes = p.a_rows * 128, sub_bytes = a_bytes + bn * 128, stage_bytes = ksub * sub_bytes;

  unsigned char* own = p.peers.base[rank];
  uint32_t* epochs = reinterpret_cast<uint32_t*>(own + kCellEpochOff);
  uint32_t* broken = reinterpret_cast<uint32_t*>(own + kBrokenOff);

  const int ntn = p.n / bn, ntm = (p.m + BM - 1) / BM, tiles = ntn * ntm;
  const int nkb = (p.k + BK - 1) / BK;
  const bool has_work = b < tiles;

  if (tid == 0) {
    *s_epoch = epochs[b] + 1;
    *s_broken = *reinterpret_cast<volatile uint32_t*>(broken) != 0;
    *abort_flag = 0;
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(bar(i), i == ACC_FREE ? 4u : 1u);
    mbar_fence_init();
    prefetch_tmap(&maps.x[mi]);
    prefetch_tmap(&maps.w[mi]);
  }
  const uint32_t tmem_cols = bn < 32 ? 32u : static_cast<uint32_t>(bn);
  if (warp == 5 && has_work) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t e = *s_epoch;
  if (!has_work) {  // nothing to compute: the call is still counted
    if (tid == 0) epochs[b] = e;
    return;
  }
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0, use = 0;  // ring position: stage and how often it has been used
      bool ok = true;
      for (int t = b; t < tiles && ok; t += p.nblocks) {
        const int mt = t / ntn, nt = t - mt * ntn;
        for (int kb = 0; kb < nkb; kb += ksub) {
          if (use > 0 && !(ok = wait_or_abort(bar(EMPTY0 + s), (use - 1) & 1, abort_flag))) break;
          // every sub-tile is fetched, also past the end of k: those arrive as zeros and add nothing
          mbar_expect_tx(bar(FULL0 + s), stage_bytes);
          const uint32_t dst = ring + s * stage_bytes;
          for (int j = 0; j < ksub; ++j) {
            tma_load_3d(dst + j * sub_bytes, &maps.x[mi], bar(FULL0 + s), (kb + j) * BK, 0, mt * BM);
            tma_load_3d(dst + j * sub_bytes + a_bytes, &maps.w[mi], bar(FULL0 + s), (kb + j) * BK, 0, nt * bn);
          }
          if (++s == NST) {
            s = 0;
            ++use;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, bn, 0, 0);
      const uint64_t desc0 = umma_desc(ring, 16, 1024);
      int s = 0, use = 0, i = 0;
      bool ok = true;
      for (int t = b; t < tiles && ok; t += p.nblocks, ++i) {
        // the accumulator is overwritten: the previous tile must have been read out
        if (i > 0 && !(ok = wait_or_abort(bar(ACC_FREE), (i - 1) & 1, abort_flag))) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; kb += ksub) {
          if (!(ok = wait_or_abort(bar(FULL0 + s), use & 1, abort_flag))) break;
          tc_fence_after();
          const uint64_t da = desc0 + static_cast<uint64_t>((s * stage_bytes) >> 4);
          const uint64_t db = da + static_cast<uint64_t>(a_bytes >> 4);
          for (int j = 0; j < ksub; ++j) {
            const uint64_t off = static_cast<uint64_t>((j * sub_bytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks)
              umma_ss(tmem, da + off + 2 * ks, db + off + 2 * ks, idesc, (kb > 0 || j > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar(EMPTY0 + s));  // the stage is free once these products have read it
          if (++s == NST) {
            s = 0;
            ++use;
          }
        }
        if (ok) umma_commit(bar(ACC_FULL));
      }
      if (!ok) {  // nothing may still be running on TMEM when it is freed
        umma_commit(bar(DRAIN));
        (void)mbar_wait(bar(DRAIN), 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue = all-reduce
    const int r = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int64_t ct = 32 * static_cast<int64_t>(bn);  // cells of one tile
    const int64_t area1 = kHeaderBytes + (2 + static_cast<int64_t>(e & 1)) * p.stage_bytes;  // [tile slot][source][cell]
    const int64_t area2 = kHeaderBytes + (6 + static_cast<int64_t>(e & 1)) * p.stage_bytes;  // [tile][cell]
    bool gave_up = *s_broken != 0;
    // a cell of this call, or (after the clock limit) whatever is there
    auto wait_cell = [&](const uint4* src, uint4 v) {
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
    auto store_row = [&](int t, int ch, const uint32_t (&res)[16]) {  // 32 columns of this thread's output row
      const int mt = t / ntn, nt = t - mt * ntn;
      uint4* dst = reinterpret_cast<uint4*>(p.out[mi] + static_cast<int64_t>(mt * BM + r) * p.out_stride + nt * bn + ch * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(res[4 * q], res[4 * q + 1], res[4 * q + 2], res[4 * q + 3]);
    };

    auto store_cell = [&](int t, int c, uint32_t lo, uint32_t hi) {  // 4 columns of this thread's output row
      const int mt = t / ntn, nt = t - mt * ntn;
      *reinterpret_cast<uint2*>(p.out[mi] + static_cast<int64_t>(mt * BM + r) * p.out_stride + nt * bn + c * 4) = make_uint2(lo, hi);
    };
    const int64_t ctw = ct / w;  // two shots: cells of a tile that one rank owns

    int i = 0;
    bool ok = true;
    for (int t = b; t < tiles && ok; t += p.nblocks, ++i) {
      const int mt = t / ntn;
      const bool valid = mt * BM + r < p.m;
      if (!(ok = wait_or_abort(bar(ACC_FULL), i & 1, abort_flag))) break;
      tc_fence_after();
      for (int ch = 0; ch < bn / 32; ++ch) {
        uint32_t v[32];
        __syncwarp();  // lanes leave the previous chunk's cell waits at different times
        tmem_ld32(tmem + lane_addr + ch * 32, v);
        tmem_wait_ld();
        if (ch == bn / 32 - 1) {  // the accumulator is in registers: the next tile may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(ACC_FREE));
        }
        uint32_t pk[16];  // this rank's partial, rounded to bf16 as the unfused projection would
#pragma unroll
        for (int q = 0; q < 16; ++q) pk[q] = pack_bf16x2(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
        if (!valid) continue;
        const int64_t idx0 = static_cast<int64_t>(ch * 8) * 128 + r;  // cell (column group ch*8 + cc, row r) = idx0 + cc * 128
        if (p.one_shot) {
          // every rank sums every cell: my partial goes to every peer, region [tile][source]
          for (int k = 1; k < w; ++k) {
            const int j = (rank + k) % w;
            uint4* dst = reinterpret_cast<uint4*>(p.peers.base[j] + area1) + (static_cast<int64_t>(t) * w + rank) * ct + idx0;
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) st_volatile16(dst + cc * 128, make_uint4(pk[2 * cc], e, pk[2 * cc + 1], e));
          }
          // partials in rank order; the next source's cells are in flight while one is added
          float acc[8][4];
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) acc[cc][0] = acc[cc][1] = acc[cc][2] = acc[cc][3] = 0.f;
          const uint4* mine = reinterpret_cast<const uint4*>(own + area1) + static_cast<int64_t>(t) * w * ct + idx0;
          uint4 cur[8], nxt[8];
          auto fetch = [&](int src, uint4 (&buf)[8]) {
            if (src >= w || src == rank) return;
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) buf[cc] = ld_volatile16(mine + src * ct + cc * 128);
          };
          fetch(0, cur);
          for (int src = 0; src < w; ++src) {
            fetch(src + 1, nxt);
            if (src == rank) {
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) add4(acc[cc], pk[2 * cc], pk[2 * cc + 1]);
            } else {
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) {
                const uint4 c = wait_cell(mine + src * ct + cc * 128, cur[cc]);
                add4(acc[cc], c.x, c.z);
              }
            }
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) cur[cc] = nxt[cc];
          }
          uint32_t res[16];
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) {
            res[2 * cc] = pack_bf16x2(acc[cc][0], acc[cc][1]);
            res[2 * cc + 1] = pack_bf16x2(acc[cc][2], acc[cc][3]);
          }
          store_row(t, ch, res);
          continue;
        }
        // Two shots.  Column group c of tile t (4 columns of all 128 rows) is owned by rank
        // (t + c) mod w, so every block of every rank pushes, sums and collects the same amount.
        // First my partials of the groups other ranks own: region [tile][source][owner's k-th group].
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const int c = ch * 8 + cc, o = (t + c) % w;
          if (o != rank)
            st_volatile16(reinterpret_cast<uint4*>(p.peers.base[o] + area1) + (static_cast<int64_t>(t) * w + rank) * ctw + (c / w) * 128 + r,
                          make_uint4(pk[2 * cc], e, pk[2 * cc + 1], e));
        }
        // Then the groups I own: all sources' cells in flight at once, added in rank order.
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const int c = ch * 8 + cc;
          if ((t + c) % w != rank) continue;
          const uint4* mine = reinterpret_cast<const uint4*>(own + area1) + static_cast<int64_t>(t) * w * ctw + (c / w) * 128 + r;
          uint4 got[kMaxRanks];
#pragma unroll
          for (int src = 0; src < kMaxRanks; ++src)
            if (src < w && src != rank) got[src] = ld_volatile16(mine + src * ctw);
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int src = 0; src < kMaxRanks; ++src) {
            if (src >= w) continue;
            if (src == rank) {
              add4(acc, pk[2 * cc], pk[2 * cc + 1]);
            } else {
              const uint4 cell = wait_cell(mine + src * ctw, got[src]);
              add4(acc, cell.x, cell.z);
            }
          }
          const uint32_t lo = pack_bf16x2(acc[0], acc[1]), hi = pack_bf16x2(acc[2], acc[3]);
          for (int k = 1; k < w; ++k) {
            const int j = (rank + k) % w;  // every owner starts with another peer
            st_volatile16(reinterpret_cast<uint4*>(p.peers.base[j] + area2) + static_cast<int64_t>(t) * ct + idx0 + cc * 128,
                          make_uint4(lo, e, hi, e));
          }
          store_cell(t, c, lo, hi);
        }
      }
    }
    // two shots: the column groups that other ranks own arrive in this rank's result-cell area
    for (int t = b; t < tiles && ok && !p.one_shot; t += p.nblocks) {
      const int mt = t / ntn;
      if (mt * BM + r >= p.m) continue;
      const uint4* results = reinterpret_cast<const uint4*>(own + area2) + static_cast<int64_t>(t) * ct + r;
      for (int ch = 0; ch < bn / 32; ++ch) {
        uint4 c[8];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc)
          if ((t + ch * 8 + cc) % w != rank) c[cc] = ld_volatile16(results + (ch * 8 + cc) * 128);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          if ((t + ch * 8 + cc) % w == rank) continue;
          c[cc] = wait_cell(results + (ch * 8 + cc) * 128, c[cc]);
          store_cell(t, ch * 8 + cc, c[cc].x, c[cc].z);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (*abort_flag) atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
    epochs[b] = e;
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// How a problem is run.  bn: the smallest of 32 / 64 / 128 columns that leaves at most one tile per
// thread block (128 wide otherwise).  one_shot: every rank pushes its partial of every tile to
// every peer and sums for itself -- one NVLink crossing instead of two, (w-1) x the bytes; chosen
// by the rule of the plain all-reduce (always at two ranks, at more up to kCellsOneShotMaxBytes
// of output) where the cell area holds a region per tile and source.
// mode: 0 = that rule, 1 = one shot where it fits, 2 = two shots.  bn == 0: the shape or the cell
// areas do not allow the kernel.
struct Plan {
  int bn = 0, a_rows = 0, ksub = 0, nst = 0, one_shot = 0;
};
static Plan make_plan(int64_t m, int64_t n, int64_t k, int world, int64_t stage_bytes, int nblocks, int mode) {
  Plan pl;
  if (m <= 0 || n <= 0 || k <= 0 || k % 8 || n % 32 || world < 2 || world > kMaxRanks) return pl;
  const int64_t ntm = (m + BM - 1) / BM;
  int bn = 0;
  for (int c = 32; c <= 128; c *= 2) {
    if (n % c) break;
    bn = c;
    if (ntm * (n / c) <= nblocks) break;
  }
  if (!bn) return pl;
  const int64_t tiles = ntm * (n / bn), cell_bytes = 32 * static_cast<int64_t>(bn) * 16;
  const bool one_fits = tiles * world * cell_bytes <= stage_bytes;
  // two shots: a tile's 4-column groups are dealt out to the ranks in turn (8 groups at bn = 32)
  const bool two_fits = (world == 2 || world == 4 || world == 8) && tiles * cell_bytes <= stage_bytes;
  const bool one_preferred = world == 2 || m * n * 2 <= kCellsOneShotMaxBytes;
  if (one_fits && (mode == 1 || (mode == 0 && one_preferred) || !two_fits)) pl.one_shot = 1;
  else if (!two_fits) return pl;
  pl.bn = bn;
  pl.a_rows = ntm > 1 ? BM : static_cast<int>((m + 15) / 16 * 16);
  const int sub = (pl.a_rows + bn) * 128;
  pl.ksub = sub <= 12 * 1024 ? 4 : sub <= 24 * 1024 ? 2 : 1;
  const int stage = sub * pl.ksub;
  pl.nst = RING_BYTES / stage < MAX_NST ? RING_BYTES / stage : MAX_NST;
  return pl;
}
static int mode_from_env() {  // measurement aid, read on every call; the same on every rank
  const char* s = std::getenv("NVLLM_GEMM_AR_MODE");
  const int v = s ? std::atoi(s) : 0;
  return v >= 0 && v <= 2 ? v : 0;
}

static int prepare_kernel() {
  static bool attr_done[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_NO_DEVICE, "ar_gemm_allreduce: no CUDA device is usable");
  }
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(NVLLM_E_CUDA, "ar_gemm_allreduce: set-up failed: %s", cudaGetErrorString(e));
    }
    attr_done[dev] = true;
  }
  return NVLLM_OK;
}

}  // namespace gar
}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_ar_gemm_tile(int64_t m, int64_t n, int64_t k, int32_t world, int64_t max_bytes) {
  return gar::make_plan(m, n, k, world, max_bytes, ar::kGrid, gar::mode_from_env()).bn;
}

extern "C" int nvllm_ar_gemm_allreduce(const void* x, int64_t x_stride, const void* weight, int64_t w_stride, void* out,
                                       int64_t out_stride, int64_t m, int64_t n, int64_t k, void* stream) {
  ar::State* s = ar::current_state();
  if (!s || !s->connected) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce: not connected (nvllm_ar_init + nvllm_ar_connect first)");
  if (m == 0) return NVLLM_OK;
  if (!x || !weight || !out) return fail(NVLLM_E_NULL, "ar_gemm_allreduce: NULL pointer argument");
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || x_stride % 8 || w_stride % 8 || out_stride % 8)
    return fail(NVLLM_E_ALIGN, "ar_gemm_allreduce: pointers and row strides must be 16-byte aligned");
  if (x_stride < k || w_stride < k || out_stride < n) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce: a row stride is shorter than its row");
  const gar::Plan pl = gar::make_plan(m, n, k, s->world, s->stage_bytes, ar::kGrid, gar::mode_from_env());
  const int bn = pl.bn;
  if (!bn)
    return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce: m=%lld n=%lld k=%lld does not fit (n %% 32, k %% 8, at least one tile per rank, %lld-byte cell areas)",
                (long long)m, (long long)n, (long long)k, (long long)s->stage_bytes);
  if (int rc = gar::prepare_kernel()) return rc;
  gar::Maps maps;
  if (!sm100::make_tmap_3d(&maps.x[0], x, k, 1, m, k, x_stride, pl.a_rows)) return NVLLM_E_CUDA;
  if (!sm100::make_tmap_3d(&maps.w[0], weight, k, 1, n, k, w_stride, bn)) return NVLLM_E_CUDA;
  gar::Params p{};
  p.out[0] = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.bn = bn;
  p.a_rows = pl.a_rows;
  p.ksub = pl.ksub;
  p.nst = pl.nst;
  p.one_shot = pl.one_shot;
  p.rank = s->rank;
  p.world = s->world;
  p.nblocks = ar::kGrid;
  p.stage_bytes = s->stage_bytes;
  p.wait_cycles = s->wait_cycles;
  p.peers = s->peers;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "ar_gemm_allreduce: no CUDA device is usable");
  gar::gemm_allreduce_kernel<<<ar::kGrid, gar::NTHREADS, gar::SMEM, static_cast<cudaStream_t>(stream)>>>(maps, p);
  count_launch();
  return check_launch("ar_gemm_allreduce launch");
}

extern "C" int nvllm_ar_gemm_allreduce_emulated(int32_t world, const void* const* xs, const void* const* weights, void* const* outputs,
                                                int64_t m, int64_t n, int64_t k, void* scratch, int64_t scratch_bytes,
                                                int64_t max_bytes, int32_t mode, void* stream) {
  if (world < 2 || world > ar::kMaxRanks) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce_emulated: world=%d invalid", world);
  if (!xs || !weights || !outputs || !scratch) return fail(NVLLM_E_NULL, "ar_gemm_allreduce_emulated: NULL pointer argument");
  if (max_bytes <= 0 || max_bytes % 16) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce_emulated: max_bytes invalid");
  if (scratch_bytes < static_cast<int64_t>(world) * (ar::kHeaderBytes + ar::kAreas * max_bytes) || !aligned16(scratch))
    return fail(NVLLM_E_WORKSPACE, "ar_gemm_allreduce_emulated: scratch too small or misaligned");
  if (mode < 0 || mode > 2) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce_emulated: mode=%d invalid", mode);
  const gar::Plan pl = gar::make_plan(m, n, k, world, max_bytes, ar::kEmulatedGrid, mode);
  const int bn = pl.bn;
  if (!bn) return fail(NVLLM_E_GEOMETRY, "ar_gemm_allreduce_emulated: m=%lld n=%lld k=%lld does not fit", (long long)m, (long long)n, (long long)k);
  if (int rc = gar::prepare_kernel()) return rc;
  gar::Maps maps;
  gar::Params p{};
  for (int r = 0; r < world; ++r) {
    if (!xs[r] || !weights[r] || !outputs[r]) return fail(NVLLM_E_NULL, "ar_gemm_allreduce_emulated: NULL pointer argument");
    if (!aligned16(xs[r]) || !aligned16(weights[r]) || !aligned16(outputs[r]))
      return fail(NVLLM_E_ALIGN, "ar_gemm_allreduce_emulated: pointers must be 16-byte aligned");
    if (!sm100::make_tmap_3d(&maps.x[r], xs[r], k, 1, m, k, k, pl.a_rows)) return NVLLM_E_CUDA;
    if (!sm100::make_tmap_3d(&maps.w[r], weights[r], k, 1, n, k, k, bn)) return NVLLM_E_CUDA;
    p.out[r] = static_cast<__nv_bfloat16*>(outputs[r]);
    p.peers.base[r] = static_cast<unsigned char*>(scratch) + r * (ar::kHeaderBytes + ar::kAreas * max_bytes);
  }
  for (int r = world; r < ar::kMaxRanks; ++r) {
    maps.x[r] = maps.x[0];
    maps.w[r] = maps.w[0];
  }
  p.out_stride = n;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.bn = bn;
  p.a_rows = pl.a_rows;
  p.ksub = pl.ksub;
  p.nst = pl.nst;
  p.one_shot = pl.one_shot;
  p.rank = -1;
  p.world = world;
  p.nblocks = ar::kEmulatedGrid;
  p.stage_bytes = max_bytes;
  p.wait_cycles = sm100::kWaitLimitCycles;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "ar_gemm_allreduce_emulated: no CUDA device is usable");
  // all ranks' blocks must be resident together (they wait on each other): a cooperative launch
  // refuses to start otherwise
  void* args[] = {&maps, &p};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gar::gemm_allreduce_kernel), dim3(ar::kEmulatedGrid * world),
                                              dim3(gar::NTHREADS), args, gar::SMEM, static_cast<cudaStream_t>(stream));
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_CUDA, "ar_gemm_allreduce_emulated launch: %s", cudaGetErrorString(e));
  }
  return NVLLM_OK;
}

