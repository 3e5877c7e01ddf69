// Varlen causal GQA prefill on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head_dim
// 64 or 128.  Math follows the prefill branch of nanovllm/layers/attention.py:67-73
// (flash_attn_varlen_func, causal, optional block table).
//
// Tile pipeline: 128 query rows x 64-key tiles; S = Q K^T (SS form, both operands K-major in
// shared memory) into one of two S buffers in TMEM; the softmax warps (thread = query row) read
// their row of S with tcgen05.ld, write P as packed bf16 over it with tcgen05.st; O += P V (TS
// form: P from TMEM, V as an MN-major shared-memory operand); Q, K, V arrive by TMA tile loads
// (128-byte swizzle, no multicast) into a two-stage ring; one tcgen05.commit per MMA group.
// Twelve warps: 0-3 softmax / correction (thread = query row), 4-7 epilogue (same rows: when an
// item's last P V product is done they normalise O and store it while the softmax warps are
// already in the next item's first tile), warp 8 lane 0 = TMA producer, warp 9 lane 0 = MMA issuer;
// the three warp groups trade registers at start-up (setmaxnreg) so that two such blocks fit an
// SM.  A thread block does not end with its query tile: two blocks per SM stay resident
// for the whole launch, keep their TMEM allocation and barriers, and pull work items (sequence,
// query tile, head group) from a global counter.  Under grouped-query attention the 128 rows of a tile are
// 128/n tokens x n query heads that share a KV head (n = 1, 2, 4 or 8), not 128 tokens of one
// head: the causal diagonal and the ragged end of a sequence then cut through a narrower band
// of tokens, so fewer of the issued products are masked or padding.  What this buys on short prompts, where a block only has a handful of
// key tiles: the block launch / TMEM allocation / barrier set-up is paid once, the producer
// lane fetches the next item and starts its Q and first K loads while the current item is
// still in its last softmax, and the tensor pipe runs the next item's first S product under
// the current item's epilogue.
//
// Order of the items: sequences longest first (ranked in shared memory by every block at start-up,
// for batches of up to SORT_BATCH sequences), a sequence's long tiles first, head groups fastest.
// The blocks that are still busy when the counter runs out are then working on the cheapest
// items, so the launch ends without a tail of half-idle SMs.
//
// Item hand-off: the producer lane decodes an item into one of two descriptor slots in shared
// memory (ITEM_FULL / ITEM_FREE barriers).  All rings keep running across items: tile t of the
// block's life uses stage t&1 and barrier phase (t>>1)&1, so the next item's first K/V tiles
// are fetched under the current item's last products.  The first P V product of an item waits
// for the previous item's O to be read (O_FREE); the softmax warps leave each row's 1 / sum in
// shared memory (EPI_FULL) and move on.  The epilogue needs no block-wide buffer: an epilogue
// warp owns the same 32 rows in TMEM and in the output, and passes them 32 columns at a time
// through a private 2 KB patch of shared memory to turn row-per-lane registers into 64-byte row
// segments.
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "prefill.cuh"
#include "prefill_tc.cuh"
#include "sm100.cuh"

namespace nvllm {
using namespace sm100;

namespace tcp {
using namespace tc;
constexpr int MAX_BATCH = kPrefillMaxBatch;  // prefix array of query tiles per sequence lives in shared memory
constexpr int SORT_BATCH = 256;  // batches up to this size are ranked by length (B^2 / 192 compares per thread)
enum PBar {
  ITEM_FULL0 = tc::NUM_BARS, ITEM_FULL1, ITEM_FREE0, ITEM_FREE1, O_FREE, EPI_FULL0, EPI_FULL1, P_NUM_BARS
};
// Twelve warps in three groups of four: softmax, epilogue, and (TMA producer, MMA issuer, two idle).
// Registers are handed over between the groups at start-up (setmaxnreg): two blocks of 384 threads
// per SM leave 80 per thread at launch; the softmax rows need about twice that, the other groups
// a fraction.  128 x (RS + RE + RX) = 384 x 80.
constexpr int NTHREADS_P = 384;
constexpr int REGS_SOFTMAX = 136, REGS_EPILOGUE = 64, REGS_OTHER = 40;
static_assert(128 * (REGS_SOFTMAX + REGS_EPILOGUE + REGS_OTHER) <= 384 * 80, "register pool of a block");
// Shared-memory layout and tile sizes for one head_dim (64 or 128).  A tile row is split into
// 64-element (128-byte) sub-tiles, the unit of the 128-byte swizzle.
template <int D_>
struct Geo {
  static constexpr int D = D_;
  static constexpr int NSUB = D / 64;               // sub-tiles per tile row
  static constexpr int Q_SUB = BM * 128, Q_BYTES = NSUB * Q_SUB;
  static constexpr int KV_SUB = BN * 128, KV_BYTES = NSUB * KV_SUB;
  static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + KST * KV_BYTES;
  static constexpr int OFF_STAGE = OFF_V + KST * KV_BYTES;  // 4 warps x 32 rows x 64 B of output
  static constexpr int OFF_CTRL = OFF_STAGE + 4 * 2048;     // barriers (8 B each)
  static constexpr int OFF_SLOTS = OFF_CTRL + 256;         // two item descriptors of 8 ints
  static constexpr int OFF_MISC = OFF_SLOTS + 64;          // tmem address, abort flag
  static constexpr int OFF_PREFIX = OFF_MISC + 64;         // (MAX_BATCH + 1) ints
  static constexpr int OFF_ORDER = OFF_PREFIX + (MAX_BATCH + 1) * 4 + 60;  // MAX_BATCH u16: sequences, longest first
  static constexpr int OFF_INV = OFF_ORDER + MAX_BATCH * 2;  // 2 items x 128 rows: 1 / row sum, softmax -> epilogue
  static constexpr int SMEM = OFF_INV + 2 * 128 * 4 + 1024;
  static constexpr int OCH = D / 32;      // 32-column chunks of O
  static constexpr int ROWB = D * 2;      // bytes of one output row
  static constexpr int PIECES = D / 8;    // 16-byte pieces of one row
};
constexpr int NUM_SLOTS = 64;                     // launches that may be in flight at once
static_assert(P_NUM_BARS * 8 <= 256, "barrier area");
}  // namespace tcp

// Work counters, one pair per launch slot; the last block of a launch to leave resets its pair.
__device__ unsigned int g_item_counter[tcp::NUM_SLOTS];
__device__ unsigned int g_done_counter[tcp::NUM_SLOTS];

struct Item {
  int b, h, m0, q0, Lq, k0, Lk, n_kv;  // n_kv < 0: no more work
};

template <int D>
__global__ void __launch_bounds__(tcp::NTHREADS_P, 2)
prefill_tcp_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const int counter_slot) {
  using namespace tcp;
  using G = Geo<D>;
  constexpr int Q_SUB = G::Q_SUB, KV_BYTES = G::KV_BYTES, KV_SUB = G::KV_SUB;
  constexpr int OFF_Q = G::OFF_Q, OFF_K = G::OFF_K, OFF_V = G::OFF_V, OFF_CTRL = G::OFF_CTRL;
  constexpr int OFF_SLOTS = G::OFF_SLOTS, OFF_MISC = G::OFF_MISC, OFF_PREFIX = G::OFF_PREFIX, OFF_ORDER = G::OFF_ORDER;
  constexpr int OCH = G::OCH, PIECES = G::PIECES;
  extern __shared__ unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + OFF_CTRL;
  auto bar = [&](int i) { return bars + 8u * i; };
  volatile int* slots = reinterpret_cast<volatile int*>(base_ptr + OFF_SLOTS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + OFF_MISC + 8);
  int* prefix = reinterpret_cast<int*>(base_ptr + OFF_PREFIX);  // prefix[i] = query tiles before the i-th sequence in order
  unsigned short* order = reinterpret_cast<unsigned short*>(base_ptr + OFF_ORDER);  // order[i] = i-th longest sequence
  // Head packing: the rows of a tile are BMT = 128 / n query tokens x n query heads of one KV head
  // (row = token * n + head; n = p.pack need not be a power of two: 7 heads x 18 tokens leave two
  // rows unused), so short and ragged sequences waste fewer rows above the diagonal and past
  // their end, and the packed heads share every K/V tile.
  const int pack = p.pack, BMT = BM / pack;

  // Rank the sequences by key length, longest first (ties by index): rank = how many come before.
  if (p.batch <= SORT_BATCH) {
    for (int b = tid; b < p.batch; b += NTHREADS_P) prefix[b] = p.cu_k[b + 1] - p.cu_k[b];  // lengths, for a moment
    __syncthreads();
    int my_rank[(SORT_BATCH + NTHREADS_P - 1) / NTHREADS_P];
#pragma unroll
    for (int k = 0; k < (SORT_BATCH + NTHREADS_P - 1) / NTHREADS_P; ++k) {
      const int b = tid + k * NTHREADS_P;
      int rank = 0;
      if (b < p.batch) {
        const int mine = prefix[b];
        for (int o = 0; o < p.batch; ++o) {
          const int theirs = prefix[o];
          rank += (theirs > mine) || (theirs == mine && o < b);
        }
      }
      my_rank[k] = rank;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < (SORT_BATCH + NTHREADS_P - 1) / NTHREADS_P; ++k) {
      const int b = tid + k * NTHREADS_P;
      if (b < p.batch) order[my_rank[k]] = static_cast<unsigned short>(b);
    }
  } else {
    for (int b = tid; b < p.batch; b += NTHREADS_P) order[b] = static_cast<unsigned short>(b);
  }
  __syncthreads();
  if (warp == 8) {
    // query tiles per sequence, in that order -> exclusive prefix sum (warp scan, 32 at a time)
    int carry = 0;
    for (int i0 = 0; i0 < p.batch; i0 += 32) {
      const int i = i0 + lane;
      int tiles = 0;
      if (i < p.batch) {
        const int b = order[i];
        tiles = (p.cu_q[b + 1] - p.cu_q[b] + BMT - 1) / BMT;
      }
      int incl = tiles;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      if (i < p.batch) prefix[i] = carry + incl - tiles;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      prefix[p.batch] = carry;
      for (int i = 0; i < P_NUM_BARS; ++i) {
        // four softmax warps fill P and the normalisers; four epilogue warps free O; an item slot is
        // free when the softmax warps, the epilogue warps and the MMA issuer are done with it
        const uint32_t count = (i == P_FULL0 || i == P_FULL1 || i == O_FREE || i == EPI_FULL0 || i == EPI_FULL1) ? 4u
                               : (i == ITEM_FREE0 || i == ITEM_FREE1)                                               ? 9u
                                                                                                                    : 1u;
        mbar_init(bar(i), count);
      }
      *abort_flag = 0;
      mbar_fence_init();
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
    }
  }
  if (warp == 9) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 128;

  auto read_item = [&](int it) {
    volatile int* s = slots + (it & 1) * 8;
    Item x;
    x.b = s[0]; x.h = s[1]; x.m0 = s[2]; x.q0 = s[3];
    x.Lq = s[4]; x.k0 = s[5]; x.Lk = s[6]; x.n_kv = s[7];
    return x;
  };

  float* inv_buf = reinterpret_cast<float*>(base_ptr + G::OFF_INV);
  // The register hand-over sits inside each group's own branch: the allocator bounds the code that
  // follows a setmaxnreg on its path, and paths that merged again would all get the smallest bound.
  if (warp >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHER));
   if (warp == 8) {
    // ------------------------------------------------------------------ producer lane
    if (lane == 0) {
      const int hgroups = p.hq / pack;
      const int total_items = prefix[p.batch] * hgroups;
      int T = 0;   // key tiles loaded so far in this block's life
      int nq = 0;  // items with at least one key tile so far (Q_FULL phase)
      // Item number -> item: (query tile of a sequence, head); heads vary fastest so that the blocks
      // working side by side share K/V tiles in L2.
      auto decode_item = [&](unsigned idx) {
        Item x;
        while (true) {
          x.n_kv = -1;
          if (idx >= static_cast<unsigned>(total_items)) break;
          const int pi = idx / hgroups;
          x.h = (idx - pi * hgroups) * pack;  // first of the packed heads
          int lo = 0, hi = p.batch;  // largest i with prefix[i] <= pi
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= pi) lo = mid; else hi = mid;
          }
          x.b = order[lo];
          x.q0 = p.cu_q[x.b];
          x.Lq = p.cu_q[x.b + 1] - x.q0;
          x.k0 = p.cu_k[x.b];
          x.Lk = p.cu_k[x.b + 1] - x.k0;
          const int tiles = prefix[lo + 1] - prefix[lo];
          x.m0 = (tiles - 1 - (pi - prefix[lo])) * BMT;  // a sequence's long tiles first
          const int kv_end = min(x.Lk, min(x.m0 + BMT, x.Lq) + (x.Lk - x.Lq));
          x.n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;
          if (x.n_kv > 0) break;
          // No visible key for the whole tile (only possible when Lk < Lq, which the engine
          // never produces): the rows are zero; written here, the other roles never see it.
          for (int r = x.m0; r < min(x.m0 + BMT, x.Lq); ++r) {
            uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(x.q0 + r) * p.out_stride + x.h * D);
            for (int c = 0; c < PIECES * pack; ++c) dst[c] = make_uint4(0, 0, 0, 0);  // the packed heads are adjacent
          }
          idx = atomicAdd(&g_item_counter[counter_slot], 1u);
        }
        return x;
      };
      // The counter is read a little ahead of need -- when the loads of the current item's last
      // three key tiles are about to be issued -- so that the round trip of the atomic runs under
      // the end of the current item instead of in front of the next one.  Not earlier: an item
      // reserved long before its block is free is an item that an idle block cannot take (measured:
      // reserving at the start of the current item cost 9 % on four 4096-token sequences).
      unsigned next_idx = atomicAdd(&g_item_counter[counter_slot], 1u);
      for (int it = 0;; ++it) {
        const Item x = decode_item(next_idx);
        if (it >= 2 && !wait_or_abort(bar(ITEM_FREE0 + (it & 1)), ((it >> 1) - 1) & 1, abort_flag)) break;
        volatile int* s = slots + (it & 1) * 8;
        s[0] = x.b; s[1] = x.h; s[2] = x.m0; s[3] = x.q0;
        s[4] = x.Lq; s[5] = x.k0; s[6] = x.Lk; s[7] = x.n_kv;
        mbar_arrive(bar(ITEM_FULL0 + (it & 1)));
        if (x.n_kv < 0) break;

        const int kvh = x.h / p.g;
        // Q buffer: free once the last S product of the previous item is complete
        if (T > 0 && !wait_or_abort(bar(QK_DONE0 + ((T - 1) & 1)), ((T - 1) >> 1) & 1, abort_flag)) break;
        mbar_expect_tx(bar(Q_FULL), G::NSUB * pack * BMT * 128);  // the box holds pack x BMT rows per sub-tile
        tma_load_3d(base + OFF_Q, &tmap_q, bar(Q_FULL), 0, x.h, x.q0 + x.m0);
        if constexpr (G::NSUB == 2) tma_load_3d(base + OFF_Q + Q_SUB, &tmap_q, bar(Q_FULL), 64, x.h, x.q0 + x.m0);
        ++nq;
        const int32_t* bt_row = p.block_tables ? p.block_tables + x.b * p.bt_stride : nullptr;
        bool ok = true;
        for (int j = 0; j < x.n_kv; ++j) {
          if (j == max(0, x.n_kv - 3)) next_idx = atomicAdd(&g_item_counter[counter_slot], 1u);
          const int t = T + j, st = t & 1, use = t >> 1;
          int row;
          if (bt_row) {
            int64_t blk = bt_row[(j * BN) / kBlockSize];
            if (blk < 0 || blk >= p.num_blocks) {
              atomicOr(p.status, NVLLM_STATUS_BAD_BLOCK);
              blk = 0;
            }
            row = static_cast<int>(blk * kBlockSize + (j * BN) % kBlockSize);
          } else {
            row = x.k0 + j * BN;
          }
          if (use > 0 && !(ok = wait_or_abort(bar(QK_DONE0 + st), (use - 1) & 1, abort_flag))) break;
          mbar_expect_tx(bar(K_FULL0 + st), KV_BYTES);
          tma_load_3d(base + OFF_K + st * KV_BYTES, &tmap_k, bar(K_FULL0 + st), 0, kvh, row);
          if constexpr (G::NSUB == 2) tma_load_3d(base + OFF_K + st * KV_BYTES + KV_SUB, &tmap_k, bar(K_FULL0 + st), 64, kvh, row);
          if (use > 0 && !(ok = wait_or_abort(bar(PV_DONE0 + st), (use - 1) & 1, abort_flag))) break;
          mbar_expect_tx(bar(V_FULL0 + st), KV_BYTES);
          tma_load_3d(base + OFF_V + st * KV_BYTES, &tmap_v, bar(V_FULL0 + st), 0, kvh, row);
          if constexpr (G::NSUB == 2) tma_load_3d(base + OFF_V + st * KV_BYTES + KV_SUB, &tmap_v, bar(V_FULL0 + st), 64, kvh, row);
        }
        if (!ok) break;
        T += x.n_kv;
      }
    }
   } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(BM, D, 0, 1);
      const uint64_t q_desc = umma_desc(base + OFF_Q, 16, 1024);
      const uint64_t k_desc = umma_desc(base + OFF_K, 16, 1024);
      const uint64_t v_desc = umma_desc(base + OFF_V, KV_SUB, 1024);
      auto issue_qk = [&](int t) -> bool {
        const int st = t & 1;
        if (!wait_or_abort(bar(K_FULL0 + st), (t >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint64_t kd = k_desc + static_cast<uint64_t>(st * (KV_BYTES >> 4));
        const uint32_t d_tmem = tmem + st * 64;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t qoff = ((ks >> 2) * Q_SUB + (ks & 3) * 32) >> 4;
          const uint64_t koff = ((ks >> 2) * KV_SUB + (ks & 3) * 32) >> 4;
          umma_ss(d_tmem, q_desc + qoff, kd + koff, idesc_qk, ks > 0);
        }
        umma_commit(bar(QK_DONE0 + st));
        return true;
      };
      int T = 0, nq = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        if (!(ok = wait_or_abort(bar(ITEM_FULL0 + (it & 1)), (it >> 1) & 1, abort_flag))) break;
        const Item x = read_item(it);
        if (x.n_kv < 0) break;
        if (!(ok = wait_or_abort(bar(Q_FULL), nq & 1, abort_flag))) break;
        ++nq;
        if (!(ok = issue_qk(T))) break;
        for (int j = 0; j < x.n_kv; ++j) {
          const int t = T + j, st = t & 1, ph = (t >> 1) & 1;
          if (j + 1 < x.n_kv && !(ok = issue_qk(t + 1))) break;  // next S runs under this tile's softmax
          if (!(ok = wait_or_abort(bar(V_FULL0 + st), ph, abort_flag))) break;
          if (!(ok = wait_or_abort(bar(P_FULL0 + st), ph, abort_flag))) break;
          // the first product of an item overwrites O: the previous item's O must have been read
          if (j == 0 && it > 0 && !(ok = wait_or_abort(bar(O_FREE), (it - 1) & 1, abort_flag))) break;
          tc_fence_after();
          const uint64_t vd = v_desc + static_cast<uint64_t>(st * (KV_BYTES >> 4));
          const uint32_t p_tmem = tmem + st * 64;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            umma_ts(tmem_o, p_tmem + ks * 8, vd + static_cast<uint64_t>((ks * 2048) >> 4), idesc_pv,
                    (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(bar(PV_DONE0 + st));
        }
        if (!ok) break;
        T += x.n_kv;
        mbar_arrive(bar(ITEM_FREE0 + (it & 1)));
      }
      if (!ok) {  // make sure nothing is still running on TMEM before it is freed
        umma_commit(bar(DRAIN));
        (void)mbar_wait(bar(DRAIN), 0);
      }
    }
   }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ softmax rows
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    const int r = warp * 32 + lane;
    const int r_tok = r / pack;  // this row's token within the tile (== BMT for the unused rows of a 7-head tile)
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    int T = 0;
    bool ok = true;
    for (int it = 0; ok; ++it) {
      if (!(ok = wait_or_abort(bar(ITEM_FULL0 + (it & 1)), (it >> 1) & 1, abort_flag))) break;
      const Item x = read_item(it);
      if (x.n_kv < 0) break;
      const int qi = x.m0 + r_tok, off = x.Lk - x.Lq;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < x.n_kv; ++j) {
        const int t = T + j, st = t & 1, ph = (t >> 1) & 1;
        const uint32_t tmem_s = tmem + st * 64 + lane_addr;
        if (!(ok = wait_or_abort(bar(QK_DONE0 + st), ph, abort_flag))) break;
        tc_fence_after();
        uint32_t s[64];
        tmem_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_wait_ld();

        const int j0 = j * BN;
        if ((j0 + BN - 1 > x.m0 + off) || (j0 + BN > x.Lk)) {  // tile touches the diagonal or the end
          const int limit = min(qi + off, x.Lk - 1) - j0;        // columns c <= limit are visible
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c > limit) s[c] = 0xff800000u;  // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 64; c += 8) {
          mx4[0] = fmax3(mx4[0], __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
          mx4[1] = fmax3(mx4[1], __uint_as_float(s[c + 2]), __uint_as_float(s[c + 3]));
          mx4[2] = fmax3(mx4[2], __uint_as_float(s[c + 4]), __uint_as_float(s[c + 5]));
          mx4[3] = fmax3(mx4[3], __uint_as_float(s[c + 6]), __uint_as_float(s[c + 7]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_new = fmaxf(m_used, mx * p.scale_log2e);
        // lazy rescale: keep the old reference maximum unless it has been outgrown by 2^8
        const bool grow = m_new > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          float alpha = 1.f;
          if (grow) {
            alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
            m_used = m_new;
            l *= alpha;
          }
          if (j > 0) {  // O holds tiles 0..j-1 of this item once the previous P V product has finished
            if (!(ok = wait_or_abort(bar(PV_DONE0 + ((t - 1) & 1)), ((t - 1) >> 1) & 1, abort_flag))) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < OCH; ++c) {
              uint32_t o[32];
              tmem_ld32(tmem_o + lane_addr + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tmem_st32(tmem_o + lane_addr + c * 32, o);
            }
          }
        }
        const float msub = (m_used == -INFINITY) ? 0.f : m_used;
        // p = 2^(s * scale - m): the multiply-subtract and the row sum run two lanes at a time
        const uint64_t scale2 = pack2(p.scale_log2e, p.scale_log2e), nmsub2 = pack2(-msub, -msub);
        uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 32; ++c) {  // P is packed in place: s[c] <- (p[2c], p[2c+1])
          float a0, a1;
          unpack2(fma2(pack2(__uint_as_float(s[2 * c]), __uint_as_float(s[2 * c + 1])), scale2, nmsub2), a0, a1);
          const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
          sum2[c & 1] = add2(sum2[c & 1], pack2(p0, p1));
          s[c] = pack_bf16x2(p0, p1);
        }
        {
          float t0, t1, t2, t3;
          unpack2(sum2[0], t0, t1);
          unpack2(sum2[1], t2, t3);
          l += (t0 + t1) + (t2 + t3);
        }
        if (j0 + BN > x.Lk) {
          // Last tile of the sequence: V rows past the end hold whatever the cache block (or the
          // next sequence) has there.  Their P is 0, but 0 x NaN would still poison O, so the
          // rows are cleared in shared memory before the product is issued.
          if (!(ok = wait_or_abort(bar(V_FULL0 + st), ph, abort_flag))) break;
          const int first = x.Lk - j0;  // rows [first, 64) are dead
          unsigned char* vt = base_ptr + OFF_V + st * KV_BYTES;
          for (int i = r; i < (BN - first) * PIECES; i += 128) {
            const int row = first + i / PIECES, piece = i % PIECES;
            *reinterpret_cast<uint4*>(vt + (piece >> 3) * KV_SUB + row * 128 + (piece & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async();
        }
        tmem_st32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FULL0 + st));
      }
      if (!ok) break;
      T += x.n_kv;

      // the row's normaliser goes to the epilogue warps; this warp is done with the item
      inv_buf[(it & 1) * 128 + r] = l > 0.f ? 1.f / l : 0.f;
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(EPI_FULL0 + (it & 1)));
        mbar_arrive(bar(ITEM_FREE0 + (it & 1)));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue rows
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_EPILOGUE));
    // Same rows as softmax warp (warp - 4): a warp reaches the TMEM lanes 32 x (warp mod 4).
    const int ew = warp - 4, r = ew * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(ew * 32) << 16;
    unsigned char* stage = base_ptr + G::OFF_STAGE + ew * 2048;  // this warp's 32 rows x 64 B
    int T = 0;
    bool ok = true;
    for (int it = 0; ok; ++it) {
      if (!(ok = wait_or_abort(bar(ITEM_FULL0 + (it & 1)), (it >> 1) & 1, abort_flag))) break;
      const Item x = read_item(it);
      if (x.n_kv < 0) break;
      T += x.n_kv;
      if (!(ok = wait_or_abort(bar(EPI_FULL0 + (it & 1)), (it >> 1) & 1, abort_flag))) break;
      const float inv = inv_buf[(it & 1) * 128 + r];
      // epilogue: O / l -> bf16; 32 columns at a time through this warp's patch of shared memory
      if (!(ok = wait_or_abort(bar(PV_DONE0 + ((T - 1) & 1)), ((T - 1) >> 1) & 1, abort_flag))) break;
      tc_fence_after();
      // lane -> (row, 16-byte piece) of the eight 64-byte row segments one store instruction writes
      const int srow = lane >> 2, spiece = lane & 3;
      __nv_bfloat16* out_tile = p.out + static_cast<int64_t>(x.q0 + x.m0) * p.out_stride + x.h * D;
      const int toks_valid = min(BMT, x.Lq - x.m0);
#pragma unroll
      for (int c = 0; c < OCH; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_addr + c * 32, o);
        tmem_wait_ld();
        if (c == OCH - 1) {  // O is in registers: the next item's first product may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(O_FREE));
        }
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[k].x = pack_bf16x2(__uint_as_float(o[8 * k]) * inv, __uint_as_float(o[8 * k + 1]) * inv);
          v[k].y = pack_bf16x2(__uint_as_float(o[8 * k + 2]) * inv, __uint_as_float(o[8 * k + 3]) * inv);
          v[k].z = pack_bf16x2(__uint_as_float(o[8 * k + 4]) * inv, __uint_as_float(o[8 * k + 5]) * inv);
          v[k].w = pack_bf16x2(__uint_as_float(o[8 * k + 6]) * inv, __uint_as_float(o[8 * k + 7]) * inv);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(stage + lane * 64 + ((k ^ ((lane >> 1) & 3)) << 4)) = v[k];
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int lr = i * 8 + srow;       // row within the warp's 32
          const int row = ew * 32 + lr;      // row of the tile
          const int tok = row / pack, hh = row - tok * pack;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + lr * 64 + ((spiece ^ ((lr >> 1) & 3)) << 4));
          if (tok < toks_valid)
            *reinterpret_cast<uint4*>(out_tile + static_cast<int64_t>(tok) * p.out_stride + hh * D + c * 32 + spiece * 8) = v;
        }
        __syncwarp();
      }
      if (lane == 0) mbar_arrive(bar(ITEM_FREE0 + (it & 1)));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (*abort_flag) atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
    // the last block to leave re-arms this launch slot's counters
    if (atomicAdd(&g_done_counter[counter_slot], 1u) == gridDim.x - 1) {
      g_item_counter[counter_slot] = 0;
      g_done_counter[counter_slot] = 0;
      __threadfence();
    }
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------

template <int D>
static int launch_prefill_tcp_t(const PrefillParams& p_in, int64_t total_q, int64_t total_k, cudaStream_t stream) {
  using G = tcp::Geo<D>;
  static bool attr_done[64] = {false};
  static std::atomic<unsigned> launch_seq{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(NVLLM_E_NO_DEVICE, "prefill: device index %d out of range", dev);
  if (p_in.out_stride > (1 << 23)) return fail(NVLLM_E_GEOMETRY, "prefill: out row stride %lld too large", (long long)p_in.out_stride);
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tcp_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
    if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "prefill (persistent): set-up failed: %s", cudaGetErrorString(e));
    // The warp groups trade registers inside the pool the block gets at launch (threads x the kernel's
    // register count); a build whose count is below the assumed 80 could never satisfy the softmax
    // group's request, and that request waits without a bound.
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, prefill_tcp_kernel<D>);
    if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "prefill (persistent): set-up failed: %s", cudaGetErrorString(e));
    if (attr.numRegs * tcp::NTHREADS_P < 128 * (tcp::REGS_SOFTMAX + tcp::REGS_EPILOGUE + tcp::REGS_OTHER))
      return fail(NVLLM_E_CUDA, "prefill (persistent): built with %d registers per thread, the warp groups' hand-over needs %d",
                  attr.numRegs, 128 * (tcp::REGS_SOFTMAX + tcp::REGS_EPILOGUE + tcp::REGS_OTHER) / tcp::NTHREADS_P);
    attr_done[dev] = true;
  }
  // heads packed into a query tile: the largest divisor of the group size that is at most 8
  // (NVLLM_PREFILL_PACK = 1..8 caps it; measurement aid, read on every call)
  int cap = 8;
  if (const char* s = std::getenv("NVLLM_PREFILL_PACK")) cap = std::atoi(s);
  PrefillParams p = p_in;
  p.pack = 1;
  for (int n = 2; n <= 8 && n <= cap; ++n)
    if (p.g % n == 0) p.pack = n;
  const int pack = p.pack, bmt = tc::BM / pack;
  CUtensorMap mq, mk, mv;
  if (!make_tmap_3d(&mq, p.q, D, p.hq, total_q, D, p.q_stride, bmt, pack)) return NVLLM_E_CUDA;
  if (p.block_tables) {
    const uint64_t slots = static_cast<uint64_t>(p.num_blocks) * kBlockSize;
    const uint64_t row = static_cast<uint64_t>(p.hkv) * D;
    if (!make_tmap_3d(&mk, p.k, D, p.hkv, slots, D, row, tc::BN)) return NVLLM_E_CUDA;
    if (!make_tmap_3d(&mv, p.v, D, p.hkv, slots, D, row, tc::BN)) return NVLLM_E_CUDA;
  } else {
    if (!make_tmap_3d(&mk, p.k, D, p.hkv, total_k, D, p.k_stride, tc::BN)) return NVLLM_E_CUDA;
    if (!make_tmap_3d(&mv, p.v, D, p.hkv, total_k, D, p.v_stride, tc::BN)) return NVLLM_E_CUDA;
  }
  // an upper bound of the work items known to the host: no more blocks than that
  const int64_t max_items = static_cast<int64_t>((p.max_seqlen_q + bmt - 1) / bmt) * (p.hq / pack) * p.batch;
  int grid = 2 * num_sms();
  if (grid <= 0) return fail(NVLLM_E_NO_DEVICE, "prefill: no CUDA device is usable");
  if (max_items < grid) grid = static_cast<int>(max_items);
  // the two head_dim instantiations share the counter array: give each its own half
  const int slot = static_cast<int>(launch_seq.fetch_add(1) % (tcp::NUM_SLOTS / 2)) + (D == 64 ? tcp::NUM_SLOTS / 2 : 0);
  prefill_tcp_kernel<D><<<grid, tcp::NTHREADS_P, G::SMEM, stream>>>(p, mq, mk, mv, slot);
  count_launch();
  return check_launch("prefill (tcgen05, persistent) launch");
}

int launch_prefill_tcp(const PrefillParams& p, int64_t total_q, int64_t total_k, cudaStream_t stream) {
  if (p.d == 128) return launch_prefill_tcp_t<128>(p, total_q, total_k, stream);
  return launch_prefill_tcp_t<64>(p, total_q, total_k, stream);
}

}  // namespace nvllm
