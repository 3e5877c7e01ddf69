// Paged GQA decode attention (one query token per sequence) for sm_100a.
//
// Math follows the decode branch of nanovllm/layers/attention.py:74-77
// (flash_attn_with_kvcache over a block table): out[b,h] = softmax(scale q.K^T) V over the
// first context_lens[b] cached tokens, query head h reading KV head h / G.  The step variant
// also does what store_kvcache does just before it (attention.py:65-66) for the one new token
// of every sequence.
//
// Design (HBM-bandwidth bound; every cached byte is read exactly once, by a fixed set of
// resident thread blocks that all finish together):
//   * The batch is cut into work units of UNIT = NW x TT tokens (64 for head_dim 128).  The
//     units of all sequences, in batch order, form one list; it is split into `n_ranges` equal
//     contiguous ranges, and thread block (range s, KV head g) streams range s of KV head g.
//     The grid is n_ranges x Hkv = two blocks per SM, a function of host-visible sizes only, so
//     the launch can be captured in a CUDA graph.  Every block derives the split from
//     context_lens itself (a block-wide scan of the units per sequence), so blocks carry the
//     same number of bytes whatever the lengths are: no tail of half-empty waves, one ramp-up.
//   * A thread block has NW warps that do not synchronise with one another while streaming.
//     Warp w owns the TT-token tile w of every unit and runs its own NST-stage cp.async ring
//     (16-byte copies, XOR-swizzled rows so ldmatrix is conflict free).  The ring keeps running
//     across sequence boundaries.  Rows past the end of a context are zero-filled, never read.
//   * Tensor cores do the dot products with the tokens on the M side so that G <= 8 query
//     heads fit the N=8 side without padding M: S^T[16 tok x 8 heads] = K[16 x D] Q^T[D x 8]
//     and O^T[D x 8] += V^T[D x 16] P^T[16 x 8] (mma.sync.m16n8k16, bf16 in / fp32 out).
//     The softmax statistics of a head are reduced over the 8 token lanes by warp shuffles.
//   * When a range leaves a sequence, the NW warps merge their (max, sum, O) through a
//     dedicated patch of shared memory.  A sequence that lies inside one range is normalised
//     and written as bf16 at once.  A sequence cut by a range boundary gives one fp32 partial
//     per range; the block that delivers the last partial (an arrival counter per (sequence,
//     KV head) in the workspace, no waiting) merges them in range order and writes the row, so
//     there is no second launch.  The counters are returned to zero by that block.
//   * Step variant: the block that streams token ctx-1 of a sequence takes that row from the
//     new K/V activation instead of the cache and writes it to its cache slot on the way.
#include <cstdlib>

#include "common.cuh"

// Pipeline shape of the head_dim-128 kernel: tokens per warp tile, ring stages per warp, warps per
// block (overridable at build time for sweeps; the defaults are the measured best).
#ifndef NVLLM_DEC_TT
#define NVLLM_DEC_TT 16
#endif
#ifndef NVLLM_DEC_NST
#define NVLLM_DEC_NST 3
#endif
#ifndef NVLLM_DEC_NW
#define NVLLM_DEC_NW 4
#endif

namespace nvllm {

// Workspace layout: [arrival counters: kCounterSlots u32][partials O][partials (max, sum)].
// The counter area has one fixed size so that calls of different geometries can share one
// workspace: whatever a call leaves in the partial area, the counters are all zero again.
constexpr int kCounterSlots = 16384;  // batch * Hkv must not exceed this
constexpr int64_t kCounterBytes = static_cast<int64_t>(kCounterSlots) * 4;
constexpr int kMaxDecodeCtas = 1024;  // the workspace is sized for at most this many thread blocks

struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  __nv_bfloat16* k_cache;  // written only by the step variant
  __nv_bfloat16* v_cache;
  const int32_t* ctx_lens;
  const int32_t* block_tables;
  int64_t bt_stride;
  int max_blocks;
  __nv_bfloat16* out;
  int64_t out_stride;
  int batch, hq, hkv, g;
  float scale_log2e;
  int64_t num_blocks;
  // step variant: the new token's rows; k_new == nullptr for plain decode
  const __nv_bfloat16* k_new;
  int64_t k_new_stride;
  const __nv_bfloat16* v_new;
  int64_t v_new_stride;
  const int32_t* slot_mapping;
  int n_ranges;
  unsigned int* counters;  // [batch * hkv], zero between launches
  float* ws_o;             // [n_ranges + batch][hq][D]
  float* ws_ml;            // [n_ranges + batch][hq][2] = (running max in log2 units, sum)
  int* status;
};

template <int D_, int TT_, int NST_, int NW_>
struct DecodeCfg {
  static constexpr int D = D_, TT = TT_, NST = NST_, NW = NW_;
  static constexpr int UNIT = NW * TT;               // tokens per work unit
  static constexpr int CPR = D / 8;                  // 16-byte pieces per row
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int TILE_BYTES = TT * ROW_BYTES;  // one tensor, one stage
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int WARP_BYTES = NST * STAGE_BYTES;
  static constexpr int RING_BYTES = NW * WARP_BYTES;
  static constexpr int MERGE_BYTES = NW * 8 * D * 4 + NW * 8 * 2 * 4;
  static constexpr int SMEM = RING_BYTES + MERGE_BYTES;
  static constexpr int MT = TT / 16;  // 16-token MMA row tiles per warp tile
  static constexpr int KS = D / 16;   // k-steps of the QK^T product
  static constexpr int DT = D / 16;   // 16-row tiles of O^T
  static_assert(TT % 16 == 0 && kBlockSize % TT == 0, "a warp tile must not straddle a cache block");
  static_assert((TT * CPR) % 32 == 0, "tile copy must divide evenly over a warp");
};

// The sequence a block is working in: index, global index of its first unit, units, length.
struct SeqCursor {
  int b, first, units, ctx;
};

template <class C>
__global__ void __launch_bounds__(C::NW * 32, 2) decode_paged_kernel(const DecodeParams p) {
  constexpr int D = C::D, TT = C::TT, NST = C::NST, NW = C::NW, UNIT = C::UNIT, NT = NW * 32;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_scan[NW];
  __shared__ int s_start[2];
  __shared__ int s_last_arrival;

  pdl_prologue();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int kvh = blockIdx.x % p.hkv;
  const int range = blockIdx.x / p.hkv;
  const int ctx_cap = p.max_blocks * kBlockSize;
  auto length_of = [&](int b) {
    const int c = p.ctx_lens[b];
    return c < 0 ? 0 : (c > ctx_cap ? ctx_cap : c);
  };
  auto units_of = [](int ctx) { return (ctx + UNIT - 1) / UNIT; };

  // ---- 1. units per sequence, block-wide scan, this block's range of the unit list ------
  const int per_thread = (p.batch + NT - 1) / NT;
  const int b_lo = min(tid * per_thread, p.batch), b_hi = min(b_lo + per_thread, p.batch);
  int local = 0;
  for (int b = b_lo; b < b_hi; ++b) {
    const int c = length_of(b);
    local += units_of(c);
    if (c == 0 && b % p.n_ranges == range) {  // empty context: defined output (zeros), no cache access
      uint4* dst = reinterpret_cast<uint4*>(p.out + b * p.out_stride + static_cast<int64_t>(kvh * p.g) * D);
      for (int i = 0; i < p.g * D / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  int incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    if (w < warp) before += s_scan[w];
    total += s_scan[w];
  }
  const int excl = before + incl - local;
  // No more ranges than units, so that every range in use holds at least one unit and the
  // ranges that share a sequence are consecutive.
  const int n_ranges = min(p.n_ranges, total);
  if (range >= n_ranges) return;  // block-uniform (also when the whole batch is empty)
  const int u0 = static_cast<int>(static_cast<int64_t>(total) * range / n_ranges);
  const int u1 = static_cast<int>(static_cast<int64_t>(total) * (range + 1) / n_ranges);
  if (local > 0 && excl <= u0 && u0 < excl + local) {  // the one thread whose sequences hold unit u0
    int first = excl;
    for (int b = b_lo;; ++b) {
      const int n = units_of(length_of(b));
      if (u0 < first + n) {
        s_start[0] = b;
        s_start[1] = first;
        break;
      }
      first += n;
    }
  }
  __syncthreads();
  // the range that holds global unit u (ranges are [total*s/n, total*(s+1)/n))
  auto range_of = [&](int u) {
    return static_cast<int>((static_cast<int64_t>(u + 1) * n_ranges - 1) / total);
  };

  SeqCursor cc;  // compute side
  cc.b = s_start[0];
  cc.first = s_start[1];
  cc.ctx = length_of(cc.b);
  cc.units = units_of(cc.ctx);
  SeqCursor pc = cc;  // load side, NST-1 units ahead
  auto seek = [&](SeqCursor& c, int u) {  // u < total, so c.b stays inside the batch
    while (u >= c.first + c.units) {
      c.first += c.units;
      ++c.b;
      c.ctx = length_of(c.b);
      c.units = units_of(c.ctx);
    }
  };

  // Q^T as the B operand: lane (gid, tig) holds q[head gid][16*ks + 2*tig .. +1] and [.. + 8].
  auto load_q = [&](uint32_t (&dst)[C::KS][2], int b) {
    const __nv_bfloat16* qrow = p.q + b * p.q_stride + static_cast<int64_t>(kvh * p.g + gid) * D;
#pragma unroll
    for (int ks = 0; ks < C::KS; ++ks) {
      if (gid < p.g) {
        dst[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * tig);
        dst[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * tig);
      } else {
        dst[ks][0] = 0u;
        dst[ks][1] = 0u;
      }
    }
  };
  uint32_t qb[C::KS][2], qn[C::KS][2];  // this sequence's fragments; the next sequence's, fetched early
  load_q(qb, cc.b);
  int qn_b = min(cc.b + 1, p.batch - 1);
  load_q(qn, qn_b);

  const uint32_t warp_smem = smem_u32(smem) + warp * C::WARP_BYTES;
  const int64_t row_elems = static_cast<int64_t>(p.hkv) * D;

  auto load_tile = [&](const SeqCursor& c, int u, int stage) {
    const int t0 = (u - c.first) * UNIT + warp * TT;
    if (t0 >= c.ctx) return;  // this warp has no token in the sequence's last unit
    int64_t blk = p.block_tables[c.b * p.bt_stride + t0 / kBlockSize];
    const bool blk_ok = blk >= 0 && blk < p.num_blocks;
    if (!blk_ok) {
      if (lane == 0) atomicOr(p.status, NVLLM_STATUS_BAD_BLOCK);
      blk = 0;
    }
    const int64_t slot0 = blk * kBlockSize + (t0 % kBlockSize);
    // Step variant: token ctx-1 is the one being decoded.  Its row comes from the activation
    // and goes to the cache from here, provided slot_mapping agrees with the block table.
    const int last = c.ctx - 1;
    bool take_new = false;
    if (p.k_new != nullptr && last < t0 + TT) {  // last >= t0 holds because t0 < ctx
      const int32_t slot = p.slot_mapping[c.b];
      if (slot >= 0) {
        if (blk_ok && slot == slot0 + (last - t0)) take_new = true;
        else if (lane == 0) atomicOr(p.status, NVLLM_STATUS_BAD_SLOT);
      }
    }
    const uint32_t kdst = warp_smem + stage * C::STAGE_BYTES;
#pragma unroll
    for (int it = 0; it < TT * C::CPR / 32; ++it) {
      const int idx = it * 32 + lane;
      const int r = idx / C::CPR, col = idx % C::CPR;
      const int bytes = (blk_ok && t0 + r < c.ctx) ? 16 : 0;
      const int64_t off = bytes ? (slot0 + r) * row_elems + kvh * D + col * 8 : 0;
      const uint32_t dst = kdst + r * C::ROW_BYTES + ((col ^ (r & 7)) << 4);
      if (take_new && t0 + r == last) {
        const int64_t in_row = static_cast<int64_t>(kvh) * D + col * 8;
        const uint4 kk = *reinterpret_cast<const uint4*>(p.k_new + c.b * p.k_new_stride + in_row);
        const uint4 vv = *reinterpret_cast<const uint4*>(p.v_new + c.b * p.v_new_stride + in_row);
        *reinterpret_cast<uint4*>(p.k_cache + off) = kk;
        *reinterpret_cast<uint4*>(p.v_cache + off) = vv;
        st_shared16(dst, kk);
        st_shared16(dst + C::TILE_BYTES, vv);
      } else {
        cp_async16(dst, p.k_cache + off, bytes);
        cp_async16(dst + C::TILE_BYTES, p.v_cache + off, bytes);
      }
    }
  };

  float o[C::DT][4];
  float m0, m1, l0, l1;  // heads 2*tig and 2*tig+1
  auto reset_state = [&]() {
#pragma unroll
    for (int dt = 0; dt < C::DT; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    m0 = m1 = -INFINITY;
    l0 = l1 = 0.f;
  };
  reset_state();

  float* sm_o = reinterpret_cast<float*>(smem + C::RING_BYTES);  // [NW][8][D]
  float* sm_ml = sm_o + NW * 8 * D;                              // [NW][8][2]

  // Leaves sequence cc.b: merges the NW warps' states and writes the output row or a partial.
  auto flush = [&]() {
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
      l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    __syncthreads();  // the previous merge has been read by everyone
#pragma unroll
    for (int dt = 0; dt < C::DT; ++dt) {
      const int d = dt * 16 + gid;
      float* dst = sm_o + (warp * 8 + 2 * tig) * D + d;
      dst[0] = o[dt][0];
      dst[D] = o[dt][1];
      dst[8] = o[dt][2];
      dst[D + 8] = o[dt][3];
    }
    if (gid == 0) {
      sm_ml[(warp * 8 + 2 * tig) * 2 + 0] = m0;
      sm_ml[(warp * 8 + 2 * tig) * 2 + 1] = l0;
      sm_ml[(warp * 8 + 2 * tig + 1) * 2 + 0] = m1;
      sm_ml[(warp * 8 + 2 * tig + 1) * 2 + 1] = l1;
    }
    __syncthreads();
    const int r_first = range_of(cc.first), r_last = range_of(cc.first + cc.units - 1);
    const int n_parts = r_last - r_first + 1;  // ranges that hold a piece of this sequence
    for (int idx = tid; idx < p.g * D; idx += NT) {
      const int h = idx / D, d = idx % D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sm_ml[(w * 8 + h) * 2]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float mw = sm_ml[(w * 8 + h) * 2];
        const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mm);
        L += sm_ml[(w * 8 + h) * 2 + 1] * f;
        acc += sm_o[(w * 8 + h) * D + d] * f;
      }
      const int head = kvh * p.g + h;
      if (n_parts == 1) {
        p.out[cc.b * p.out_stride + static_cast<int64_t>(head) * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
      } else {
        // partial slot range + b: strictly increasing along the (range, sequence) pieces of the list
        const int64_t row = static_cast<int64_t>(range + cc.b) * p.hq + head;
        p.ws_o[row * D + d] = acc;
        if (d == 0) {
          p.ws_ml[row * 2 + 0] = mm;
          p.ws_ml[row * 2 + 1] = L;
        }
      }
    }
    if (n_parts > 1) {  // block-uniform
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const unsigned int arrived = atomicAdd(&p.counters[cc.b * p.hkv + kvh], 1u);
        s_last_arrival = arrived == static_cast<unsigned int>(n_parts - 1);
      }
      __syncthreads();
      if (s_last_arrival) {  // every piece is in the workspace: merge them in range order
        __threadfence();
        for (int idx = tid; idx < p.g * D; idx += NT) {
          const int h = idx / D, d = idx % D;
          const int head = kvh * p.g + h;
          const int64_t row0 = static_cast<int64_t>(r_first + cc.b) * p.hq + head;
          float mm = -INFINITY;
          for (int j = 0; j < n_parts; ++j) mm = fmaxf(mm, __ldcg(p.ws_ml + (row0 + static_cast<int64_t>(j) * p.hq) * 2));
          float L = 0.f, acc = 0.f;
          for (int j = 0; j < n_parts; ++j) {
            const int64_t row = row0 + static_cast<int64_t>(j) * p.hq;
            const float mj = __ldcg(p.ws_ml + row * 2);
            const float f = (mj == -INFINITY) ? 0.f : fast_exp2(mj - mm);
            L += __ldcg(p.ws_ml + row * 2 + 1) * f;
            acc += __ldcg(p.ws_o + row * D + d) * f;
          }
          p.out[cc.b * p.out_stride + static_cast<int64_t>(head) * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
        }
        if (tid == 0) p.counters[cc.b * p.hkv + kvh] = 0u;  // ready for the next launch
      }
    }
  };

  // ---- 2. stream the range ------------------------------------------------------------------
  const int n_units = u1 - u0;
#pragma unroll
  for (int j = 0; j < NST - 1; ++j) {
    if (j < n_units) {
      seek(pc, u0 + j);
      load_tile(pc, u0 + j, j);
    }
    cp_async_commit();
  }

  for (int i = 0;; ++i) {
    const int u = u0 + i;
    if (i == n_units || u >= cc.first + cc.units) {  // block-uniform: the range leaves sequence cc.b
      flush();
      if (i == n_units) break;
      seek(cc, u);
      reset_state();
      if (qn_b == cc.b) {
#pragma unroll
        for (int ks = 0; ks < C::KS; ++ks) {
          qb[ks][0] = qn[ks][0];
          qb[ks][1] = qn[ks][1];
        }
      } else {  // empty sequences in between
        load_q(qb, cc.b);
      }
      qn_b = min(cc.b + 1, p.batch - 1);
      load_q(qn, qn_b);
    }
    cp_async_wait<NST - 2>();
    __syncwarp();
    if (i + NST - 1 < n_units) {
      seek(pc, u + NST - 1);
      load_tile(pc, u + NST - 1, (i + NST - 1) % NST);
    }
    cp_async_commit();

    const int t0 = (u - cc.first) * UNIT + warp * TT;
    if (t0 >= cc.ctx) continue;
    const int t_end = cc.ctx;
    const uint32_t kbase = warp_smem + (i % NST) * C::STAGE_BYTES;
    const uint32_t vbase = kbase + C::TILE_BYTES;

    // S^T = K Q^T
    float s[C::MT][4];
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
      s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
      const int r = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < C::KS; ++ks) {
        const int c = ks * 2 + (lane >> 4);
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(a0, a1, a2, a3, kbase + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4));
        mma_bf16_16816(s[mt], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
      }
    }

    // scale into log2 units, mask the tail, running max / sum per head
    const bool tail = t0 + TT > t_end;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] *= p.scale_log2e;
      if (tail) {
        const int tr = t0 + mt * 16 + gid;
        if (tr >= t_end) s[mt][0] = s[mt][1] = -INFINITY;
        if (tr + 8 >= t_end) s[mt][2] = s[mt][3] = -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[mt][0], s[mt][2]));
      mx1 = fmaxf(mx1, fmaxf(s[mt][1], s[mt][3]));
    }
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: the tile has >= 1 live token
    const float alpha0 = fast_exp2(m0 - mn0), alpha1 = fast_exp2(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
      s[mt][0] = fast_exp2(s[mt][0] - mn0);
      s[mt][1] = fast_exp2(s[mt][1] - mn1);
      s[mt][2] = fast_exp2(s[mt][2] - mn0);
      s[mt][3] = fast_exp2(s[mt][3] - mn1);
      ps0 += s[mt][0] + s[mt][2];
      ps1 += s[mt][1] + s[mt][3];
    }
    l0 = l0 * alpha0 + ps0;  // per-lane partial sums; reduced over the token lanes at the flush
    l1 = l1 * alpha1 + ps1;
#pragma unroll
    for (int dt = 0; dt < C::DT; ++dt) {
      o[dt][0] *= alpha0;
      o[dt][1] *= alpha1;
      o[dt][2] *= alpha0;
      o[dt][3] *= alpha1;
    }

    // O^T += V^T P^T
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
      const uint32_t pb0 = movmatrix_trans(pack_bf16x2(s[mt][0], s[mt][1]));
      const uint32_t pb1 = movmatrix_trans(pack_bf16x2(s[mt][2], s[mt][3]));
      const int r = mt * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int dt = 0; dt < C::DT; ++dt) {
        const int c = dt * 2 + ((lane >> 3) & 1);
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4_trans(a0, a1, a2, a3, vbase + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4));
        mma_bf16_16816(o[dt], a0, a1, a2, a3, pb0, pb1);
      }
    }
  }
  cp_async_wait<0>();
}

// ---- host side -------------------------------------------------------------------------

static int env_int(const char* name, int dflt) {
  const char* s = std::getenv(name);
  if (!s || !*s) return dflt;
  return std::atoi(s);
}

// Thread blocks of a launch: two per SM of the current device (NVLLM_DECODE_CTAS, read once per
// process, overrides the total for measurements), at most kMaxDecodeCtas; with no usable device
// the cap itself, so that the sizing functions work on any host.
static int decode_ctas() {
  static const int forced = env_int("NVLLM_DECODE_CTAS", 0);
  int n = forced > 0 ? forced : 2 * num_sms();
  if (n <= 0 || n > kMaxDecodeCtas) n = kMaxDecodeCtas;
  return n;
}
static int ranges_for(int ctas, int hkv) {
  const int n = ctas / hkv;
  return n < 1 ? 1 : n;
}
static int unit_tokens(int d) { return d == 128 ? NVLLM_DEC_NW * NVLLM_DEC_TT : 4 * 32; }

static int check_decode_geometry(const char* who, int batch, int max_blocks, int hq, int hkv, int d) {
  if (d != 64 && d != 128) return fail(NVLLM_E_GEOMETRY, "%s: head_dim=%d unsupported (64 or 128)", who, d);
  if (hq <= 0 || hkv <= 0 || hq % hkv) return fail(NVLLM_E_GEOMETRY, "%s: Hq=%d must be a positive multiple of Hkv=%d", who, hq, hkv);
  if (hq / hkv > 8) return fail(NVLLM_E_GEOMETRY, "%s: group size Hq/Hkv=%d > 8 unsupported", who, hq / hkv);
  if (batch < 0 || max_blocks <= 0) return fail(NVLLM_E_GEOMETRY, "%s: batch=%d max_blocks=%d invalid", who, batch, max_blocks);
  if (static_cast<int64_t>(batch) * hkv > kCounterSlots)
    return fail(NVLLM_E_GEOMETRY, "%s: batch*Hkv=%lld exceeds the %d (sequence, KV head) pairs of one launch", who,
                (long long)batch * hkv, kCounterSlots);
  // the unit list of a launch is indexed with 32-bit integers
  const int64_t max_units = (static_cast<int64_t>(max_blocks) * kBlockSize + unit_tokens(d) - 1) / unit_tokens(d);
  if (static_cast<int64_t>(max_blocks) * kBlockSize > 0x7fffffffLL || max_units * (batch > 0 ? batch : 1) > 0x3fffffffLL)
    return fail(NVLLM_E_GEOMETRY, "%s: batch=%d x max_blocks=%d too large", who, batch, max_blocks);
  return NVLLM_OK;
}

// Counter area plus one partial per (range, sequence) piece of the unit list; there are fewer
// than ranges + batch pieces.  Sized for the cap on thread blocks, not for the device at hand.
static int64_t workspace_bytes_for(int batch, int hq, int hkv, int d) {
  if (batch == 0) return 0;
  const int64_t rows = (static_cast<int64_t>(ranges_for(kMaxDecodeCtas, hkv)) + batch) * hq;
  return kCounterBytes + rows * d * 4 + rows * 2 * 4;
}

template <class C>
static int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_paged_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "decode_paged: cannot reserve %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int grid = p.n_ranges * p.hkv;
  cudaError_t e = launch_kernel(decode_paged_kernel<C>, dim3(static_cast<unsigned>(grid)), dim3(C::NW * 32), C::SMEM, stream,
                                pdl_enabled(), p);
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_CUDA, "decode_paged launch: %s", cudaGetErrorString(e));
  }
  return NVLLM_OK;
}

// Shared body of nvllm_decode_paged and nvllm_decode_step.
static int decode_common(const char* who, const void* q, int64_t q_row_stride, const void* k_new, int64_t k_new_row_stride,
                         const void* v_new, int64_t v_new_row_stride, const int32_t* slot_mapping, void* k_cache,
                         void* v_cache, const int32_t* context_lens, const int32_t* block_tables, int64_t bt_row_stride,
                         int32_t max_blocks, void* out, int64_t out_row_stride, int32_t batch, int32_t num_q_heads,
                         int32_t num_kv_heads, int32_t head_dim, float scale, int64_t num_blocks, void* workspace,
                         int64_t workspace_bytes, void* stream, bool with_store) {
  int rc = check_decode_geometry(who, batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  if (batch == 0) return NVLLM_OK;
  if (!q || !k_cache || !v_cache || !context_lens || !block_tables || !out)
    return fail(NVLLM_E_NULL, "%s: NULL pointer argument", who);
  if (num_blocks <= 0) return fail(NVLLM_E_GEOMETRY, "%s: num_blocks=%lld must be positive", who, (long long)num_blocks);
  const int64_t qrow = static_cast<int64_t>(num_q_heads) * head_dim;
  const int64_t kvrow = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (q_row_stride < qrow || out_row_stride < qrow || bt_row_stride < max_blocks)
    return fail(NVLLM_E_GEOMETRY, "%s: a row stride is smaller than its row", who);
  if (q_row_stride % 8 || out_row_stride % 8 || !aligned16(q) || !aligned16(out) || !aligned16(k_cache) || !aligned16(v_cache))
    return fail(NVLLM_E_ALIGN, "%s: q/out/cache pointers and row strides must be 16-byte aligned", who);
  if (with_store) {
    if (!k_new || !v_new || !slot_mapping) return fail(NVLLM_E_NULL, "%s: NULL pointer argument", who);
    if (k_new_row_stride < kvrow || v_new_row_stride < kvrow)
      return fail(NVLLM_E_GEOMETRY, "%s: key/value row stride smaller than Hkv*D", who);
    if (k_new_row_stride % 8 || v_new_row_stride % 8 || !aligned16(k_new) || !aligned16(v_new))
      return fail(NVLLM_E_ALIGN, "%s: key/value pointers and row strides must be 16-byte aligned", who);
  }
  const int64_t need = workspace_bytes_for(batch, num_q_heads, num_kv_heads, head_dim);
  if (!workspace || workspace_bytes < need)
    return fail(NVLLM_E_WORKSPACE, "%s: workspace of %lld bytes needed, %lld given", who, (long long)need,
                (long long)(workspace ? workspace_bytes : 0));
  if (!aligned16(workspace)) return fail(NVLLM_E_ALIGN, "%s: workspace must be 16-byte aligned", who);

  DecodeParams p;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "%s: no CUDA device is usable", who);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_row_stride;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.ctx_lens = context_lens;
  p.block_tables = block_tables;
  p.bt_stride = bt_row_stride;
  p.max_blocks = max_blocks;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_row_stride;
  p.batch = batch;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.g = num_q_heads / num_kv_heads;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.num_blocks = num_blocks;
  p.k_new = with_store ? static_cast<const __nv_bfloat16*>(k_new) : nullptr;
  p.k_new_stride = k_new_row_stride;
  p.v_new = with_store ? static_cast<const __nv_bfloat16*>(v_new) : nullptr;
  p.v_new_stride = v_new_row_stride;
  p.slot_mapping = slot_mapping;
  p.n_ranges = ranges_for(decode_ctas(), num_kv_heads);
  const int64_t rows = (static_cast<int64_t>(ranges_for(kMaxDecodeCtas, num_kv_heads)) + batch) * num_q_heads;
  p.counters = static_cast<unsigned int*>(workspace);
  p.ws_o = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kCounterBytes);
  p.ws_ml = p.ws_o + rows * head_dim;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_decode<DecodeCfg<128, NVLLM_DEC_TT, NVLLM_DEC_NST, NVLLM_DEC_NW>>(p, st);
  return launch_decode<DecodeCfg<64, 32, 3, 4>>(p, st);
}

}  // namespace nvllm

extern "C" int64_t nvllm_decode_workspace_bytes(int32_t batch, int32_t max_blocks, int32_t num_q_heads,
                                                int32_t num_kv_heads, int32_t head_dim) {
  using namespace nvllm;
  int rc = check_decode_geometry("decode_workspace_bytes", batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  return workspace_bytes_for(batch, num_q_heads, num_kv_heads, head_dim);
}

extern "C" int nvllm_decode_plan(int32_t batch, int32_t max_blocks, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t head_dim, int32_t* unit_tokens_out, int32_t* thread_blocks_out) {
  using namespace nvllm;
  int rc = check_decode_geometry("decode_plan", batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  if (unit_tokens_out) *unit_tokens_out = unit_tokens(head_dim);
  if (thread_blocks_out) *thread_blocks_out = ranges_for(decode_ctas(), num_kv_heads) * num_kv_heads;
  return NVLLM_OK;
}

extern "C" int nvllm_decode_paged(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                  const int32_t* context_lens, const int32_t* block_tables, int64_t bt_row_stride,
                                  int32_t max_blocks, void* out, int64_t out_row_stride, int32_t batch,
                                  int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                  int64_t num_blocks, void* workspace, int64_t workspace_bytes, void* stream) {
  return nvllm::decode_common("decode_paged", q, q_row_stride, nullptr, 0, nullptr, 0, nullptr, const_cast<void*>(k_cache),
                              const_cast<void*>(v_cache), context_lens, block_tables, bt_row_stride, max_blocks, out,
                              out_row_stride, batch, num_q_heads, num_kv_heads, head_dim, scale, num_blocks, workspace,
                              workspace_bytes, stream, false);
}

extern "C" int nvllm_decode_step(const void* q, int64_t q_row_stride, const void* key, int64_t key_row_stride,
                                 const void* value, int64_t value_row_stride, const int32_t* slot_mapping, void* k_cache,
                                 void* v_cache, const int32_t* context_lens, const int32_t* block_tables,
                                 int64_t bt_row_stride, int32_t max_blocks, void* out, int64_t out_row_stride,
                                 int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                 int64_t num_blocks, void* workspace, int64_t workspace_bytes, void* stream) {
  return nvllm::decode_common("decode_step", q, q_row_stride, key, key_row_stride, value, value_row_stride, slot_mapping,
                              k_cache, v_cache, context_lens, block_tables, bt_row_stride, max_blocks, out, out_row_stride,
                              batch, num_q_heads, num_kv_heads, head_dim, scale, num_blocks, workspace, workspace_bytes,
                              stream, true);
}

// ---- decode without a caller-provided workspace ---------------------------------------------
//
// nvllm_decode_paged_static is for hosts that have no way to hand the library a scratch
// buffer: an engine that has already given all free HBM to its KV cache (nano-vllm sizes the
// cache from whatever memory is left, so a later allocation can fail), a real-time serving
// loop in which cudaMalloc's implicit device synchronisation is unacceptable, or a binding
// from a language that owns no device allocator and only forwards the pointers it was given.
// The arrival counters and the partials live in a fixed array that is part of the library image.

namespace nvllm {

constexpr int64_t kStaticScratchBytes = NVLLM_DECODE_STATIC_SCRATCH_BYTES;

// Lives in every context that loads this library, for the life of the process.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.  Like any
// file-scope device array without an initialiser it starts as zeros, which is what the
// arrival counters at its head need.
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// Device address of the array on each device, resolved on that device's first call.
static void* g_static_scratch_addr[64] = {nullptr};

static int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_NO_DEVICE, "decode_paged_static: no usable CUDA device is current");
  }
  if (!g_static_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return fail(NVLLM_E_CUDA, "decode_paged_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    }
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return NVLLM_OK;
}

}  // namespace nvllm

extern "C" int nvllm_decode_paged_static(const void* q, int64_t q_row_stride, const void* k_cache,
                                         const void* v_cache, const int32_t* context_lens,
                                         const int32_t* block_tables, int64_t bt_row_stride, int32_t max_blocks,
                                         void* out, int64_t out_row_stride, int32_t batch, int32_t num_q_heads,
                                         int32_t num_kv_heads, int32_t head_dim, float scale, int64_t num_blocks,
                                         void* stream) {
  using namespace nvllm;
  const int64_t need = nvllm_decode_workspace_bytes(batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (need < 0) return static_cast<int>(need);  // geometry rejected; message already set
  if (batch == 0) return NVLLM_OK;
  if (need > kStaticScratchBytes)
    return fail(NVLLM_E_WORKSPACE,
                "decode_paged_static: this geometry needs %lld bytes of split-KV scratch but the built-in array "
                "holds %lld; use nvllm_decode_paged with a caller-owned workspace",
                (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  // What must start at zero are the arrival counters at the head of the array.  They are zero
  // when the library is loaded, and the block that merges a sequence's partials puts its
  // counter back to zero, so every completed call leaves them cleared for the next one.  The
  // partials themselves are always written before they are read within one call.
  return nvllm_decode_paged(q, q_row_stride, k_cache, v_cache, context_lens, block_tables, bt_row_stride, max_blocks,
                            out, out_row_stride, batch, num_q_heads, num_kv_heads, head_dim, scale, num_blocks,
                            scratch, kStaticScratchBytes, stream);
}
