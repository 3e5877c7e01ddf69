// Varlen causal GQA prefill on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// head_dim 128.
//
// Math follows the prefill branch of nanovllm/layers/attention.py:67-73
// (flash_attn_varlen_func, causal, optional block table).
//
// One thread block = one 128-row query tile of one (sequence, query head), walking the keys in
// 64-token tiles; two blocks are resident per SM (96 KB of shared memory and 256 of the 512
// TMEM columns each), so one block's softmax overlaps the other's matrix products.  Six warps
// with fixed roles:
//   warps 0-3  softmax / correction / epilogue: thread r owns query row r.  It reads its row
//              of S from TMEM (tcgen05.ld, lane = row, so max and sum need no shuffles),
//              writes P as packed bf16 back into the same TMEM columns (tcgen05.st) and,
//              when the running maximum has grown by more than 2^8, rescales its row of O.
//   warp 4     TMA producer (one lane): Q once (two 128-row x 64-column boxes), then one K
//              tile and one V tile per step (two 64 x 64 boxes each), 128-byte swizzle, into
//              a two-stage ring.
//   warp 5     MMA issuer (one lane): S_j = Q K_j^T (SS form, both operands K-major in shared
//              memory) into one of two S buffers, then O += P_j V_j (TS form: P from TMEM, V
//              as an MN-major shared-memory operand).  S_{j+1} is issued before P_j V_j so it
//              runs under the softmax of tile j; completion is signalled to mbarriers with
//              tcgen05.commit.
// Every mbarrier wait is bounded; on expiry the block records NVLLM_STATUS_TIMEOUT, all roles
// leave their loops and TMEM is freed.
#include <cstdlib>

#include "common.cuh"
#include "prefill.cuh"
#include "sm100.cuh"
#include "prefill_tc.cuh"

namespace nvllm {
using namespace sm100;

__global__ void __launch_bounds__(tc::NTHREADS, 2)
prefill_tc_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap tmap_q,
                  const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v) {
  using namespace tc;
  extern __shared__ unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int b = blockIdx.z, h = blockIdx.y, kvh = h / p.g;
  const int mtile = gridDim.x - 1 - blockIdx.x;  // long tiles first
  const int q0 = p.cu_q[b], Lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], Lk = p.cu_k[b + 1] - k0;
  const int m0 = mtile * BM;
  if (m0 >= Lq) return;
  const int off = Lk - Lq;
  int kv_end = min(Lk, min(m0 + BM, Lq) + off);
  if (kv_end < 0) kv_end = 0;
  const int n_kv = (kv_end + BN - 1) / BN;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + OFF_BAR + 8 * NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + OFF_BAR + 8 * NUM_BARS + 8);
  // Loads of K/V tile j into ring stage j&1 (producer lane only).
  const int32_t* bt_row = p.block_tables ? p.block_tables + b * p.bt_stride : nullptr;
  auto kv_row = [&](int j) -> int {
    if (!bt_row) return k0 + j * BN;
    int64_t blk = bt_row[(j * BN) / kBlockSize];
    if (blk < 0 || blk >= p.num_blocks) {
      atomicOr(p.status, NVLLM_STATUS_BAD_BLOCK);
      blk = 0;
    }
    return static_cast<int>(blk * kBlockSize + (j * BN) % kBlockSize);
  };
  auto issue_k = [&](int j, int row) {
    const int st = j & 1;
    mbar_expect_tx(bar(K_FULL0 + st), KV_BYTES);
    tma_load_3d(base + OFF_K + st * KV_BYTES, &tmap_k, bar(K_FULL0 + st), 0, kvh, row);
    tma_load_3d(base + OFF_K + st * KV_BYTES + KV_SUB, &tmap_k, bar(K_FULL0 + st), 64, kvh, row);
  };
  auto issue_v = [&](int j, int row) {
    const int st = j & 1;
    mbar_expect_tx(bar(V_FULL0 + st), KV_BYTES);
    tma_load_3d(base + OFF_V + st * KV_BYTES, &tmap_v, bar(V_FULL0 + st), 0, kvh, row);
    tma_load_3d(base + OFF_V + st * KV_BYTES + KV_SUB, &tmap_v, bar(V_FULL0 + st), 64, kvh, row);
  };
  if (warp == 4 && lane == 0) {
    // The producer lane sets up the barriers itself and starts the first loads (Q and both
    // ring stages need no hand-shake) before the block-wide sync, so their latency overlaps
    // the TMEM allocation and the other warps' start-up.
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(bar(i), (i == P_FULL0 || i == P_FULL1) ? 4u : 1u);
    *abort_flag = 0;
    mbar_fence_init();
    if (n_kv > 0) {
      mbar_expect_tx(bar(Q_FULL), Q_BYTES);
      tma_load_3d(base + OFF_Q, &tmap_q, bar(Q_FULL), 0, h, q0 + m0);
      tma_load_3d(base + OFF_Q + Q_SUB, &tmap_q, bar(Q_FULL), 64, h, q0 + m0);
      for (int j = 0; j < 2 && j < n_kv; ++j) {
        const int row = kv_row(j);
        issue_k(j, row);
        issue_v(j, row);
      }
    }
  }
  if (warp == 5) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 128;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = 2; j < n_kv; ++j) {
        const int st = j & 1, use = j >> 1;
        // K stage free once S_{j-2} is complete, V stage free once P_{j-2} V_{j-2} is complete
        const int row = kv_row(j);
        if (!wait_or_abort(bar(QK_DONE0 + st), (use - 1) & 1, abort_flag)) break;
        issue_k(j, row);
        if (!wait_or_abort(bar(PV_DONE0 + st), (use - 1) & 1, abort_flag)) break;
        issue_v(j, row);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_qk = umma_idesc(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(BM, D, 0, 1);
      // Descriptors are built once; inside the loops only their 14-bit address field moves
      // (a 64-bit add of a compile-time constant), so the single issuing thread spends a few
      // instructions per MMA instead of rebuilding 64-bit descriptors.
      const uint64_t q_desc = umma_desc(base + OFF_Q, 16, 1024);
      const uint64_t k_desc = umma_desc(base + OFF_K, 16, 1024);      // stage 0; stage 1 = + KV_BYTES
      const uint64_t v_desc = umma_desc(base + OFF_V, KV_SUB, 1024);
      // S_j = Q K_j^T into S buffer j&1
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        if (!wait_or_abort(bar(K_FULL0 + st), (j >> 1) & 1, abort_flag)) return false;
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
      bool ok = wait_or_abort(bar(Q_FULL), 0, abort_flag);
      ok = ok && issue_qk(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1, ph = (j >> 1) & 1;
        if (j + 1 < n_kv && !(ok = issue_qk(j + 1))) break;  // next S runs under this tile's softmax
        if (!(ok = wait_or_abort(bar(V_FULL0 + st), ph, abort_flag))) break;
        if (!(ok = wait_or_abort(bar(P_FULL0 + st), ph, abort_flag))) break;
        tc_fence_after();
        const uint64_t vd = v_desc + static_cast<uint64_t>(st * (KV_BYTES >> 4));
        const uint32_t p_tmem = tmem + st * 64;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)
          umma_ts(tmem_o, p_tmem + ks * 8, vd + static_cast<uint64_t>((ks * 2048) >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(bar(PV_DONE0 + st));
      }
      if (!ok) {  // make sure nothing is still running on TMEM before it is freed
        umma_commit(bar(DRAIN));
        (void)mbar_wait(bar(DRAIN), 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax rows
    const int r = warp * 32 + lane;
    const int qi = m0 + r;  // query index within the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1, ph = (j >> 1) & 1;
      const uint32_t tmem_s = tmem + st * 64 + lane_addr;
      if (!(ok = wait_or_abort(bar(QK_DONE0 + st), ph, abort_flag))) break;
      tc_fence_after();
      uint32_t s[64];
      tmem_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_wait_ld();

      const int j0 = j * BN;
      if ((j0 + BN - 1 > m0 + off) || (j0 + BN > Lk)) {  // tile touches the diagonal or the end
        const int limit = min(qi + off, Lk - 1) - j0;      // columns c <= limit are visible
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c > limit) s[c] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(s[c]));
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
        if (j > 0) {  // O holds tiles 0..j-1 once the previous P V product has finished
          if (!(ok = wait_or_abort(bar(PV_DONE0 + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_flag))) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
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
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 32; ++c) {  // P is packed in place: s[c] <- (p[2c], p[2c+1])
        const float p0 = fast_exp2(fmaf(__uint_as_float(s[2 * c]), p.scale_log2e, -msub));
        const float p1 = fast_exp2(fmaf(__uint_as_float(s[2 * c + 1]), p.scale_log2e, -msub));
        sum4[c & 3] += p0 + p1;
        s[c] = pack_bf16x2(p0, p1);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (j0 + BN > Lk) {
        // Last tile of the sequence: V rows past the end hold whatever the cache block (or the
        // next sequence) has there.  Their P is 0, but 0 x NaN would still poison O, so the
        // rows are cleared in shared memory before the product is issued.
        if (!(ok = wait_or_abort(bar(V_FULL0 + st), ph, abort_flag))) break;
        const int first = Lk - j0;  // rows [first, 64) are dead
        unsigned char* vt = base_ptr + OFF_V + st * KV_BYTES;
        for (int i = r; i < (BN - first) * 16; i += 128) {
          const int row = first + (i >> 4), piece = i & 15;
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
    // epilogue: O / l -> bf16 -> global (rows past the sequence end are not written)
    if (ok && n_kv > 0) ok = wait_or_abort(bar(PV_DONE0 + ((n_kv - 1) & 1)), ((n_kv - 1) >> 1) & 1, abort_flag);
    tc_fence_after();
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    // O / l -> bf16, staged through the Q buffer (free now) so that the global stores are
    // whole 256-byte rows per half warp instead of 32 scattered 16-byte pieces.
    unsigned char* stage = base_ptr + OFF_Q;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      if (n_kv > 0 && ok) {
        tmem_ld32(tmem_o + lane_addr + c * 32, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0u;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(o[8 * k]) * inv, __uint_as_float(o[8 * k + 1]) * inv);
        v.y = pack_bf16x2(__uint_as_float(o[8 * k + 2]) * inv, __uint_as_float(o[8 * k + 3]) * inv);
        v.z = pack_bf16x2(__uint_as_float(o[8 * k + 4]) * inv, __uint_as_float(o[8 * k + 5]) * inv);
        v.w = pack_bf16x2(__uint_as_float(o[8 * k + 6]) * inv, __uint_as_float(o[8 * k + 7]) * inv);
        const int cc = c * 4 + k;  // 16-byte piece of the row
        *reinterpret_cast<uint4*>(stage + r * 256 + ((cc ^ (r & 15)) << 4)) = v;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four softmax warps only
    __nv_bfloat16* out_tile = p.out + static_cast<int64_t>(q0 + m0) * p.out_stride + h * D;
    const int rows_valid = min(BM, Lq - m0);
#pragma unroll 4
    for (int idx = r; idx < BM * 16; idx += 128) {
      const int row = idx >> 4, cc = idx & 15;
      if (row < rows_valid)
        *reinterpret_cast<uint4*>(out_tile + static_cast<int64_t>(row) * p.out_stride + cc * 8) =
            *reinterpret_cast<const uint4*>(stage + row * 256 + ((cc ^ (row & 15)) << 4));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(p.status, NVLLM_STATUS_TIMEOUT);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- known-answer check of the building blocks --------------------------------------------
// out1 = A B^T   (SS form: A and B both K-major tiles in shared memory)
// out2 = A B     (TS form: A as packed bf16 in TMEM, B as an MN-major shared-memory tile)
// A, B: [128,128] bf16 row-major; out1, out2: [128,128] fp32.
__global__ void __launch_bounds__(160, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __nv_bfloat16* __restrict__ a, float* __restrict__ out1, float* __restrict__ out2,
                     int* __restrict__ status) {
  using namespace tc;
  extern __shared__ unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + 2 * TILE_BYTES;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + 2 * TILE_BYTES + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + 2 * TILE_BYTES + 72);
  if (tid == 0) {
    mbar_init(bar(0), 1);    // tiles landed
    mbar_init(bar(1), 1);    // SS product done
    mbar_init(bar(2), 128);  // P written
    mbar_init(bar(3), 1);    // TS product done
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t A = base, B = base + TILE_BYTES;

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), 2 * TILE_BYTES);
      tma_load_3d(A, &tmap_a, bar(0), 0, 0, 0);
      tma_load_3d(A + SUB_BYTES, &tmap_a, bar(0), 64, 0, 0);
      tma_load_3d(B, &tmap_b, bar(0), 0, 0, 0);
      tma_load_3d(B + SUB_BYTES, &tmap_b, bar(0), 64, 0, 0);
      bool ok = wait_or_abort(bar(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t koff = (ks >> 2) * SUB_BYTES + (ks & 3) * 32;
          umma_ss(tmem, umma_desc(A + koff, 16, 1024), umma_desc(B + koff, 16, 1024), umma_idesc(128, 128, 0, 0), ks > 0);
        }
        umma_commit(bar(1));
        ok = wait_or_abort(bar(2), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + 128, tmem + ks * 8, umma_desc(B + ks * 2048, SUB_BYTES, 1024), umma_idesc(128, 128, 0, 1), ks > 0);
        umma_commit(bar(3));
      }
    }
  } else {
    const int r = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    bool ok = wait_or_abort(bar(1), 0, abort_flag);
    tc_fence_after();
    if (ok) {
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_addr + c * 32, v);
        tmem_wait_ld();
        for (int e = 0; e < 32; ++e) out1[r * 128 + c * 32 + e] = __uint_as_float(v[e]);
      }
      // stage row r of A as packed bf16 pairs in TMEM columns [0,64)
      uint32_t pk[64];
      const uint32_t* arow = reinterpret_cast<const uint32_t*>(a + r * 128);
      for (int c = 0; c < 64; ++c) pk[c] = arow[c];
      tmem_st32(tmem + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st32(tmem + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(2));
      ok = wait_or_abort(bar(3), 0, abort_flag);
      tc_fence_after();
      if (ok) {
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem + 128 + lane_addr + c * 32, v);
          tmem_wait_ld();
          for (int e = 0; e < 32; ++e) out2[r * 128 + c * 32 + e] = __uint_as_float(v[e]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(status, NVLLM_STATUS_TIMEOUT);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- bounded-wait check ---------------------------------------------------------------------
// One block allocates TMEM, then a thread waits on an mbarrier that nothing ever arrives at.
// The wait must run out (about a second), set the abort flag that the other roles poll, record
// NVLLM_STATUS_TIMEOUT, and the block must still free its TMEM and end normally.
__global__ void __launch_bounds__(64, 1) wait_expiry_selftest_kernel(int* __restrict__ status, int* __restrict__ result) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 64);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  bool ok = true;
  if (tid == 0) ok = wait_or_abort(smem_u32(&bars[0]), 0, abort_flag);   // runs out on the clock
  if (tid == 32) ok = wait_or_abort(smem_u32(&bars[1]), 0, abort_flag);  // leaves early through the abort flag
  if (tid == 0) result[0] = ok ? 1 : 0;
  if (tid == 32) result[1] = ok ? 1 : 0;
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(status, NVLLM_STATUS_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem_slot, 64);
}

// ---- host side ---------------------------------------------------------------------------

template <class K>
static int opt_in_smem(K kernel, int bytes, bool* done, const char* what) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || done[dev]) return NVLLM_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "%s: cannot reserve %d bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  done[dev] = true;
  return NVLLM_OK;
}

int launch_prefill_tc(const PrefillParams& p, int64_t total_q, int64_t total_k, cudaStream_t stream) {
  static bool attr_done[64] = {false};
  int rc = opt_in_smem(prefill_tc_kernel, tc::SMEM, attr_done, "prefill (tcgen05)");
  if (rc) return rc;
  CUtensorMap mq, mk, mv;
  if (!make_tmap_3d(&mq, p.q, tc::D, p.hq, total_q, tc::D, p.q_stride, tc::BM)) return NVLLM_E_CUDA;
  if (p.block_tables) {
    const uint64_t slots = static_cast<uint64_t>(p.num_blocks) * kBlockSize;
    const uint64_t row = static_cast<uint64_t>(p.hkv) * tc::D;
    if (!make_tmap_3d(&mk, p.k, tc::D, p.hkv, slots, tc::D, row, tc::BN)) return NVLLM_E_CUDA;
    if (!make_tmap_3d(&mv, p.v, tc::D, p.hkv, slots, tc::D, row, tc::BN)) return NVLLM_E_CUDA;
  } else {
    if (!make_tmap_3d(&mk, p.k, tc::D, p.hkv, total_k, tc::D, p.k_stride, tc::BN)) return NVLLM_E_CUDA;
    if (!make_tmap_3d(&mv, p.v, tc::D, p.hkv, total_k, tc::D, p.v_stride, tc::BN)) return NVLLM_E_CUDA;
  }
  dim3 grid((p.max_seqlen_q + tc::BM - 1) / tc::BM, p.hq, p.batch);
  prefill_tc_kernel<<<grid, tc::NTHREADS, tc::SMEM, stream>>>(p, mq, mk, mv);
  count_launch();
  return check_launch("prefill (tcgen05) launch");
}

}  // namespace nvllm

extern "C" int nvllm_selftest_wait_expiry(int32_t* device_result, void* stream) {
  using namespace nvllm;
  if (!device_result) return fail(NVLLM_E_NULL, "selftest_wait_expiry: device_result is NULL");
  int* status = status_word();
  if (!status) return fail(NVLLM_E_NO_DEVICE, "selftest_wait_expiry: no CUDA device is usable");
  wait_expiry_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, device_result);
  count_launch();
  return check_launch("selftest_wait_expiry launch");
}

extern "C" int nvllm_selftest_umma(const void* a, const void* b, float* out_ss, float* out_ts, void* stream) {
  using namespace nvllm;
  if (!a || !b || !out_ss || !out_ts) return fail(NVLLM_E_NULL, "selftest_umma: NULL pointer argument");
  if (!aligned16(a) || !aligned16(b)) return fail(NVLLM_E_ALIGN, "selftest_umma: inputs must be 16-byte aligned");
  int* status = status_word();
  if (!status) return fail(NVLLM_E_NO_DEVICE, "selftest_umma: no CUDA device is usable");
  static bool attr_done[64] = {false};
  const int smem = 2 * tc::TILE_BYTES + 128 + 1024;
  int rc = opt_in_smem(umma_selftest_kernel, smem, attr_done, "selftest_umma");
  if (rc) return rc;
  CUtensorMap ma, mb;
  if (!sm100::make_tmap_3d(&ma, a, 128, 1, 128, 128, 128, 128)) return NVLLM_E_CUDA;
  if (!sm100::make_tmap_3d(&mb, b, 128, 1, 128, 128, 128, 128)) return NVLLM_E_CUDA;
  umma_selftest_kernel<<<1, 160, smem, static_cast<cudaStream_t>(stream)>>>(
      ma, mb, static_cast<const __nv_bfloat16*>(a), out_ss, out_ts, status);
  count_launch();
  return check_launch("selftest_umma launch");
}
