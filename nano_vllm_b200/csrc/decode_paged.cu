// Paged GQA decode attention (one query token per sequence) for sm_100a.
//
// Math follows the decode branch of nanovllm/layers/attention.py:74-77
// (flash_attn_with_kvcache over a block table): out[b,h] = softmax(scale q.K^T) V over the
// first context_lens[b] cached tokens, query head h reading KV head h / G.
//
// Design (HBM-bandwidth bound; every cached byte is read exactly once):
//   * Work item = (sequence b, KV head g, chunk c of `chunk_tokens` tokens).  The grid is
//     batch * Hkv * max_splits thread blocks, a function of host-visible sizes only, so the
//     launch can be captured in a CUDA graph; a block whose chunk starts past context_lens[b]
//     returns at once.
//   * A thread block has NW warps that do not synchronise with one another while streaming.
//     Warp w owns the 16-token (TT-token) tiles w, w+NW, ... of the chunk and runs its own
//     NST-stage cp.async ring (16-byte copies, XOR-swizzled rows so ldmatrix is conflict
//     free).  Rows past the end of the context are zero-filled, never read from memory.
//   * Tensor cores do the dot products with the tokens on the M side so that G <= 8 query
//     heads fit the N=8 side without padding M: S^T[16 tok x 8 heads] = K[16 x D] Q^T[D x 8]
//     and O^T[D x 8] += V^T[D x 16] P^T[16 x 8] (mma.sync.m16n8k16, bf16 in / fp32 out).
//     The softmax statistics of a head are reduced over the 8 token lanes by warp shuffles.
//   * At the end the NW warps merge their (max, sum, O) through shared memory.  A sequence
//     with a single chunk is normalised and written as bf16 directly; otherwise the block
//     writes an fp32 partial and (max, sum) to the workspace and a second kernel merges the
//     chunks.
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

struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int32_t* ctx_lens;
  const int32_t* block_tables;
  int64_t bt_stride;
  int max_blocks;
  __nv_bfloat16* out;
  int64_t out_stride;
  int batch, hq, hkv, g;
  float scale_log2e;
  int64_t num_blocks;
  int chunk, max_splits;
  float* ws_o;   // [batch, hq, max_splits, D]
  float* ws_ml;  // [batch, hq, max_splits, 2] = (running max in log2 units, sum)
  int* status;
};

template <int D_, int TT_, int NST_, int NW_>
struct DecodeCfg {
  static constexpr int D = D_, TT = TT_, NST = NST_, NW = NW_;
  static constexpr int CPR = D / 8;                  // 16-byte pieces per row
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int TILE_BYTES = TT * ROW_BYTES;  // one tensor, one stage
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int WARP_BYTES = NST * STAGE_BYTES;
  static constexpr int MERGE_BYTES = NW * 8 * D * 4 + NW * 8 * 2 * 4;
  static constexpr int SMEM = (NW * WARP_BYTES > MERGE_BYTES) ? NW * WARP_BYTES : MERGE_BYTES;
  static constexpr int MT = TT / 16;  // 16-token MMA row tiles per warp tile
  static constexpr int KS = D / 16;   // k-steps of the QK^T product
  static constexpr int DT = D / 16;   // 16-row tiles of O^T
  static_assert(TT % 16 == 0 && kBlockSize % TT == 0, "a warp tile must not straddle a cache block");
  static_assert((TT * CPR) % 32 == 0, "tile copy must divide evenly over a warp");
};

template <class C>
__global__ void __launch_bounds__(C::NW * 32) decode_paged_kernel(const DecodeParams p) {
  constexpr int D = C::D, TT = C::TT, NST = C::NST, NW = C::NW;
  extern __shared__ __align__(128) unsigned char smem[];

  pdl_prologue();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;

  int work = blockIdx.x;
  const int kvh = work % p.hkv;
  work /= p.hkv;
  const int split = work % p.max_splits;
  const int b = work / p.max_splits;

  int ctx = p.ctx_lens[b];
  const int ctx_cap = p.max_blocks * kBlockSize;
  ctx = ctx < 0 ? 0 : (ctx > ctx_cap ? ctx_cap : ctx);
  const int t_begin = split * p.chunk;
  if (t_begin >= ctx) {
    if (split == 0) {  // empty context: defined output (zeros), no cache access
      for (int i = tid; i < p.g * D; i += NW * 32)
        p.out[b * p.out_stride + static_cast<int64_t>(kvh * p.g) * D + i] = __float2bfloat16(0.f);
    }
    return;
  }
  const int t_end = min(ctx, t_begin + p.chunk);
  const int n_splits = (ctx + p.chunk - 1) / p.chunk;
  const int n_tiles = (t_end - t_begin + TT - 1) / TT;
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + NW - 1) / NW : 0;

  // Q^T as the B operand: lane (gid, tig) holds q[head gid][16*ks + 2*tig .. +1] and [.. + 8].
  uint32_t qb[C::KS][2];
  {
    const __nv_bfloat16* qrow = p.q + b * p.q_stride + static_cast<int64_t>(kvh * p.g + gid) * D;
#pragma unroll
    for (int ks = 0; ks < C::KS; ++ks) {
      if (gid < p.g) {
        qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * tig);
        qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * tig);
      } else {
        qb[ks][0] = 0u;
        qb[ks][1] = 0u;
      }
    }
  }

  const uint32_t warp_smem = smem_u32(smem) + warp * C::WARP_BYTES;
  const int32_t* bt_row = p.block_tables + b * p.bt_stride;
  const int64_t row_elems = static_cast<int64_t>(p.hkv) * D;

  auto load_tile = [&](int i, int stage) {
    const int t0 = t_begin + (warp + i * NW) * TT;
    int64_t blk = bt_row[t0 / kBlockSize];
    const bool blk_ok = blk >= 0 && blk < p.num_blocks;
    if (!blk_ok) {
      if (lane == 0) atomicOr(p.status, NVLLM_STATUS_BAD_BLOCK);
      blk = 0;
    }
    const int64_t slot0 = blk * kBlockSize + (t0 % kBlockSize);
    const uint32_t kdst = warp_smem + stage * C::STAGE_BYTES;
#pragma unroll
    for (int it = 0; it < TT * C::CPR / 32; ++it) {
      const int idx = it * 32 + lane;
      const int r = idx / C::CPR, c = idx % C::CPR;
      const int bytes = (blk_ok && t0 + r < t_end) ? 16 : 0;
      const int64_t off = bytes ? (slot0 + r) * row_elems + kvh * D + c * 8 : 0;
      const uint32_t dst = kdst + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4);
      cp_async16(dst, p.k_cache + off, bytes);
      cp_async16(dst + C::TILE_BYTES, p.v_cache + off, bytes);
    }
  };

  float o[C::DT][4];
#pragma unroll
  for (int dt = 0; dt < C::DT; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // heads 2*tig and 2*tig+1

#pragma unroll
  for (int s = 0; s < NST - 1; ++s) {
    if (s < my_tiles) load_tile(s, s);
    cp_async_commit();
  }

  for (int i = 0; i < my_tiles; ++i) {
    cp_async_wait<NST - 2>();
    __syncwarp();
    if (i + NST - 1 < my_tiles) load_tile(i + NST - 1, (i + NST - 1) % NST);
    cp_async_commit();

    const uint32_t kbase = warp_smem + (i % NST) * C::STAGE_BYTES;
    const uint32_t vbase = kbase + C::TILE_BYTES;
    const int t0 = t_begin + (warp + i * NW) * TT;

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
    l0 = l0 * alpha0 + ps0;  // per-lane partial sums; reduced over the token lanes at the end
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

#pragma unroll
  for (int sh = 4; sh <= 16; sh <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
    l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
  }

  // merge the NW warps through shared memory (staging buffers are free now)
  cp_async_wait<0>();
  __syncthreads();
  float* sm_o = reinterpret_cast<float*>(smem);          // [NW][8][D]
  float* sm_ml = sm_o + NW * 8 * D;                      // [NW][8][2]
#pragma unroll
  for (int dt = 0; dt < C::DT; ++dt) {
    const int d = dt * 16 + gid;
    float* base = sm_o + (warp * 8 + 2 * tig) * D + d;
    base[0] = o[dt][0];
    base[D] = o[dt][1];
    base[8] = o[dt][2];
    base[D + 8] = o[dt][3];
  }
  if (gid == 0) {
    sm_ml[(warp * 8 + 2 * tig) * 2 + 0] = m0;
    sm_ml[(warp * 8 + 2 * tig) * 2 + 1] = l0;
    sm_ml[(warp * 8 + 2 * tig + 1) * 2 + 0] = m1;
    sm_ml[(warp * 8 + 2 * tig + 1) * 2 + 1] = l1;
  }
  __syncthreads();

  for (int idx = tid; idx < p.g * D; idx += NW * 32) {
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
    if (n_splits == 1) {
      p.out[b * p.out_stride + static_cast<int64_t>(head) * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
    } else {
      const int64_t row = (static_cast<int64_t>(b) * p.hq + head) * p.max_splits + split;
      p.ws_o[row * D + d] = acc;
      if (d == 0) {
        p.ws_ml[row * 2 + 0] = mm;
        p.ws_ml[row * 2 + 1] = L;
      }
    }
  }
}

// Merges the split-KV partials of one (sequence, query head): grid = batch*hq, D threads.
template <int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeParams p) {
  pdl_prologue();
  const int row = blockIdx.x;
  const int b = row / p.hq, head = row % p.hq;
  int ctx = p.ctx_lens[b];
  const int ctx_cap = p.max_blocks * kBlockSize;
  ctx = ctx < 0 ? 0 : (ctx > ctx_cap ? ctx_cap : ctx);
  const int n = (ctx + p.chunk - 1) / p.chunk;
  if (n <= 1) return;  // written directly by the decode kernel
  const int d = threadIdx.x;
  const float* ml = p.ws_ml + static_cast<int64_t>(row) * p.max_splits * 2;
  const float* po = p.ws_o + static_cast<int64_t>(row) * p.max_splits * D + d;
  float mm = -INFINITY;
  for (int s = 0; s < n; ++s) mm = fmaxf(mm, ml[2 * s]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < n; ++s) {
    const float ms = ml[2 * s];
    const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mm);
    L += ml[2 * s + 1] * f;
    acc += po[static_cast<int64_t>(s) * D] * f;
  }
  p.out[b * p.out_stride + static_cast<int64_t>(head) * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

// ---- host side -------------------------------------------------------------------------

static int env_int(const char* name, int dflt) {
  const char* s = std::getenv(name);
  if (!s || !*s) return dflt;
  return std::atoi(s);
}

DecodePlan make_decode_plan(int batch, int max_blocks, int hq, int hkv, int d) {
  (void)hq;
  static const int forced_chunk = env_int("NVLLM_DECODE_CHUNK", 0);
  static const int target_ctas = env_int("NVLLM_DECODE_TARGET_CTAS", kNumSMs * 8);
  const int max_ctx = max_blocks * kBlockSize;
  const int64_t units = static_cast<int64_t>(batch) * hkv;
  int chunk;
  if (forced_chunk > 0) {
    chunk = (forced_chunk + 63) / 64 * 64;
  } else {
    // enough chunks to fill the machine, but no more than ~1 MB of KV per thread block
    const int chunk_cap = d >= 128 ? 2048 : 4096;
    const int64_t want = (target_ctas + units - 1) / units;
    int64_t c = (max_ctx + want - 1) / want;
    c = (c + kBlockSize - 1) / kBlockSize * kBlockSize;
    chunk = static_cast<int>(c < chunk_cap ? c : chunk_cap);
    // Contexts of at most 4096 tokens with at least two resident waves of (sequence, KV head)
    // units: one block per unit and no combine launch.  Measured on 256 sequences of 100-2048
    // tokens with a 4096-token table: 164 us instead of 171 us.
    if (max_ctx <= 4096 && units >= 4 * kNumSMs) chunk = max_ctx;
  }
  if (chunk > max_ctx) chunk = max_ctx;
  if (chunk < 64) chunk = 64;
  DecodePlan plan;
  plan.chunk_tokens = chunk;
  plan.max_splits = (max_ctx + chunk - 1) / chunk;
  return plan;
}

static int check_decode_geometry(const char* who, int batch, int max_blocks, int hq, int hkv, int d) {
  if (d != 64 && d != 128) return fail(NVLLM_E_GEOMETRY, "%s: head_dim=%d unsupported (64 or 128)", who, d);
  if (hq <= 0 || hkv <= 0 || hq % hkv) return fail(NVLLM_E_GEOMETRY, "%s: Hq=%d must be a positive multiple of Hkv=%d", who, hq, hkv);
  if (hq / hkv > 8) return fail(NVLLM_E_GEOMETRY, "%s: group size Hq/Hkv=%d > 8 unsupported", who, hq / hkv);
  if (batch < 0 || max_blocks <= 0) return fail(NVLLM_E_GEOMETRY, "%s: batch=%d max_blocks=%d invalid", who, batch, max_blocks);
  if (static_cast<int64_t>(max_blocks) * kBlockSize > 0x7fffffffLL) return fail(NVLLM_E_GEOMETRY, "%s: max_blocks=%d too large", who, max_blocks);
  return NVLLM_OK;
}

static int64_t workspace_bytes_for(const DecodePlan& plan, int batch, int hq, int d) {
  if (plan.max_splits <= 1) return 0;
  const int64_t rows = static_cast<int64_t>(batch) * hq * plan.max_splits;
  return rows * d * 4 + rows * 2 * 4;
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
  const int64_t grid = static_cast<int64_t>(p.batch) * p.hkv * p.max_splits;
  if (grid > 0x7fffffffLL) return fail(NVLLM_E_GEOMETRY, "decode_paged: grid too large");
  const bool pdl = pdl_enabled();
  cudaError_t e = launch_kernel(decode_paged_kernel<C>, dim3(static_cast<unsigned>(grid)), dim3(C::NW * 32), C::SMEM, stream, pdl, p);
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_CUDA, "decode_paged launch: %s", cudaGetErrorString(e));
  }
  if (p.max_splits > 1) {
    e = launch_kernel(decode_combine_kernel<C::D>, dim3(p.batch * p.hq), dim3(C::D), 0, stream, pdl, p);
    count_launch();
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(NVLLM_E_CUDA, "decode_combine launch: %s", cudaGetErrorString(e));
    }
  }
  return NVLLM_OK;
}

}  // namespace nvllm

extern "C" int64_t nvllm_decode_workspace_bytes(int32_t batch, int32_t max_blocks, int32_t num_q_heads,
                                                int32_t num_kv_heads, int32_t head_dim) {
  using namespace nvllm;
  int rc = check_decode_geometry("decode_workspace_bytes", batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  return workspace_bytes_for(make_decode_plan(batch, max_blocks, num_q_heads, num_kv_heads, head_dim), batch, num_q_heads, head_dim);
}

extern "C" int nvllm_decode_plan(int32_t batch, int32_t max_blocks, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t head_dim, int32_t* chunk_tokens, int32_t* max_splits) {
  using namespace nvllm;
  int rc = check_decode_geometry("decode_plan", batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  DecodePlan plan = make_decode_plan(batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (chunk_tokens) *chunk_tokens = plan.chunk_tokens;
  if (max_splits) *max_splits = plan.max_splits;
  return NVLLM_OK;
}

extern "C" int nvllm_decode_paged(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                  const int32_t* context_lens, const int32_t* block_tables, int64_t bt_row_stride,
                                  int32_t max_blocks, void* out, int64_t out_row_stride, int32_t batch,
                                  int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                  int64_t num_blocks, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace nvllm;
  int rc = check_decode_geometry("decode_paged", batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  if (rc) return rc;
  if (batch == 0) return NVLLM_OK;
  if (!q || !k_cache || !v_cache || !context_lens || !block_tables || !out)
    return fail(NVLLM_E_NULL, "decode_paged: NULL pointer argument");
  if (num_blocks <= 0) return fail(NVLLM_E_GEOMETRY, "decode_paged: num_blocks=%lld must be positive", (long long)num_blocks);
  const int64_t qrow = static_cast<int64_t>(num_q_heads) * head_dim;
  if (q_row_stride < qrow || out_row_stride < qrow || bt_row_stride < max_blocks)
    return fail(NVLLM_E_GEOMETRY, "decode_paged: a row stride is smaller than its row");
  if (q_row_stride % 8 || out_row_stride % 8 || !aligned16(q) || !aligned16(out) || !aligned16(k_cache) || !aligned16(v_cache))
    return fail(NVLLM_E_ALIGN, "decode_paged: q/out/cache pointers and row strides must be 16-byte aligned");

  DecodeParams p;
  const DecodePlan plan = make_decode_plan(batch, max_blocks, num_q_heads, num_kv_heads, head_dim);
  const int64_t need = workspace_bytes_for(plan, batch, num_q_heads, head_dim);
  if (need > 0) {
    if (!workspace || workspace_bytes < need)
      return fail(NVLLM_E_WORKSPACE, "decode_paged: workspace of %lld bytes needed, %lld given", (long long)need, (long long)(workspace ? workspace_bytes : 0));
    if (!aligned16(workspace)) return fail(NVLLM_E_ALIGN, "decode_paged: workspace must be 16-byte aligned");
  }
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "decode_paged: no CUDA device is usable");
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_row_stride;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
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
  p.chunk = plan.chunk_tokens;
  p.max_splits = plan.max_splits;
  const int64_t rows = static_cast<int64_t>(batch) * num_q_heads * plan.max_splits;
  p.ws_o = static_cast<float*>(workspace);
  p.ws_ml = need > 0 ? p.ws_o + rows * head_dim : nullptr;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_decode<DecodeCfg<128, NVLLM_DEC_TT, NVLLM_DEC_NST, NVLLM_DEC_NW>>(p, st);
  return launch_decode<DecodeCfg<64, 32, 3, 4>>(p, st);
}

// ---- decode without a caller-provided workspace ---------------------------------------------
//
// nvllm_decode_paged_static is for hosts that have no way to hand the library a scratch
// buffer: an engine that has already given all free HBM to its KV cache (nano-vllm sizes the
// cache from whatever memory is left, so a later allocation can fail), a real-time serving
// loop in which cudaMalloc's implicit device synchronisation is unacceptable, or a binding
// from a language that owns no device allocator and only forwards the pointers it was given.
// The split-KV partials live in a fixed array that is part of the library image.

namespace nvllm {

constexpr int64_t kStaticScratchBytes = NVLLM_DECODE_STATIC_SCRATCH_BYTES;

// Lives in every context that loads this library, for the life of the process.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
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
  if (need > kStaticScratchBytes)
    return fail(NVLLM_E_WORKSPACE,
                "decode_paged_static: this geometry needs %lld bytes of split-KV scratch but the built-in array "
                "holds %lld; use nvllm_decode_paged with a caller-owned workspace",
                (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: every partial that the combine kernel reads
  // is written by the partial kernel of the same call, so leftovers from earlier calls are
  // never observed.
  return nvllm_decode_paged(q, q_row_stride, k_cache, v_cache, context_lens, block_tables, bt_row_stride, max_blocks,
                            out, out_row_stride, batch, num_q_heads, num_kv_heads, head_dim, scale, num_blocks,
                            scratch, kStaticScratchBytes, stream);
}
