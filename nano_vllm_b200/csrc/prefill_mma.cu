// Varlen causal GQA prefill, warp-level tensor-core version (mma.sync.m16n8k16).
//
// Math follows the prefill branch of nanovllm/layers/attention.py:67-73
// (flash_attn_varlen_func, causal, optional block table): query row i of a sequence with
// Lq new tokens and Lk total tokens attends keys j <= i + (Lk - Lq).
//
// This kernel is the portable path: it serves head_dim 64 and every shape the tcgen05
// kernel declines.  One thread block = 128 query rows of one (sequence, query head), 8 warps
// of 16 rows; K/V tiles of 64 tokens are double-buffered with cp.async from either the
// packed K/V activations or the paged cache; online softmax in fp32 registers.
#include "common.cuh"
#include "prefill.cuh"

namespace nvllm {

template <int D_>
struct PrefillMmaCfg {
  static constexpr int D = D_, BM = 128, BN = 64, NW = 8;
  static constexpr int CPR = D / 8, ROW_BYTES = D * 2;
  static constexpr int Q_BYTES = BM * ROW_BYTES;
  static constexpr int KV_TILE_BYTES = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = 2 * KV_TILE_BYTES;
  static constexpr int SMEM = Q_BYTES + 2 * STAGE_BYTES;
  static constexpr int KS = D / 16, NT = BN / 8, DN = D / 8;
};

template <class C>
__global__ void __launch_bounds__(C::NW * 32) prefill_mma_kernel(const PrefillParams p) {
  constexpr int D = C::D, BM = C::BM, BN = C::BN, NTHR = C::NW * 32;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;

  const int b = blockIdx.z, h = blockIdx.y, kvh = h / p.g;
  const int mtile = gridDim.x - 1 - blockIdx.x;  // long tiles first
  const int q0 = p.cu_q[b], Lq = p.cu_q[b + 1] - q0;
  const int k0 = p.cu_k[b], Lk = p.cu_k[b + 1] - k0;
  const int m0 = mtile * BM;
  if (m0 >= Lq) return;
  const int off = Lk - Lq;
  const int m_hi = min(m0 + BM, Lq);
  int kv_end = min(Lk, m_hi + off);
  if (kv_end < 0) kv_end = 0;
  const int n_kv = (kv_end + BN - 1) / BN;

  const uint32_t q_smem = smem_u32(smem);
  const uint32_t kv_smem = q_smem + C::Q_BYTES;

  // Q tile -> shared memory (rows past Lq zero-filled)
  for (int idx = tid; idx < BM * C::CPR; idx += NTHR) {
    const int r = idx / C::CPR, c = idx % C::CPR;
    const bool ok = m0 + r < Lq;
    const __nv_bfloat16* src = ok ? p.q + static_cast<int64_t>(q0 + m0 + r) * p.q_stride + h * D + c * 8 : p.q;
    cp_async16(q_smem + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4), src, ok ? 16 : 0);
  }

  const int32_t* bt_row = p.block_tables ? p.block_tables + b * p.bt_stride : nullptr;
  auto load_kv = [&](int j, int stage) {
    const int t0 = j * BN;
    const __nv_bfloat16 *kbase, *vbase;
    int64_t kstride, vstride;
    bool tile_ok = true;
    if (bt_row) {
      int64_t blk = bt_row[t0 / kBlockSize];
      tile_ok = blk >= 0 && blk < p.num_blocks;
      if (!tile_ok) {
        if (tid == 0) atomicOr(p.status, NVLLM_STATUS_BAD_BLOCK);
        blk = 0;
      }
      const int64_t slot0 = blk * kBlockSize + t0 % kBlockSize;
      kstride = vstride = static_cast<int64_t>(p.hkv) * D;
      kbase = p.k + slot0 * kstride + kvh * D;
      vbase = p.v + slot0 * vstride + kvh * D;
    } else {
      kstride = p.k_stride;
      vstride = p.v_stride;
      kbase = p.k + static_cast<int64_t>(k0 + t0) * kstride + kvh * D;
      vbase = p.v + static_cast<int64_t>(k0 + t0) * vstride + kvh * D;
    }
    const uint32_t kdst = kv_smem + stage * C::STAGE_BYTES;
#pragma unroll
    for (int it = 0; it < BN * C::CPR / NTHR; ++it) {
      const int idx = it * NTHR + tid;
      const int r = idx / C::CPR, c = idx % C::CPR;
      const bool ok = tile_ok && t0 + r < Lk;
      const uint32_t dst = kdst + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4);
      cp_async16(dst, ok ? kbase + r * kstride + c * 8 : p.k, ok ? 16 : 0);
      cp_async16(dst + C::KV_TILE_BYTES, ok ? vbase + r * vstride + c * 8 : p.v, ok ? 16 : 0);
    }
  };

  if (n_kv > 0) load_kv(0, 0);
  cp_async_commit();

  float o[C::DN][4];
#pragma unroll
  for (int i = 0; i < C::DN; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int row_lo = m0 + warp * 16;  // first query row of this warp

  for (int j = 0; j < n_kv; ++j) {
    cp_async_wait<0>();
    __syncthreads();
    if (j + 1 < n_kv) load_kv(j + 1, (j + 1) & 1);
    cp_async_commit();

    const int t0 = j * BN;
    if (t0 > row_lo + 15 + off || row_lo >= Lq) continue;  // whole tile masked for this warp
    const uint32_t kbase = kv_smem + (j & 1) * C::STAGE_BYTES;
    const uint32_t vbase = kbase + C::KV_TILE_BYTES;

    float s[C::NT][4];
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < C::KS; ++ks) {
      uint32_t a0, a1, a2, a3;
      {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
        ldmatrix_x4(a0, a1, a2, a3, q_smem + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int np = 0; np < C::NT / 2; ++np) {
        const int r = np * 16 + (lane & 7) + (lane >> 4) * 8, c = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kbase + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4));
        mma_bf16_16816(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    const bool need_mask = (t0 + BN > row_lo + off + 1) || (t0 + BN > Lk);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * p.scale_log2e;
        if (need_mask) {
          const int jj = t0 + nt * 8 + 2 * tig + (e & 1);
          const int ii = row_lo + gid + (e >> 1) * 8;
          if (jj > ii + off || jj >= Lk) v = -INFINITY;
        }
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mn = fmaxf(mrow[r], mx[r]);
      msafe[r] = (mn == -INFINITY) ? 0.f : mn;
      alpha[r] = fast_exp2(mrow[r] - msafe[r]);
      mrow[r] = mn;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < C::NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = fast_exp2(s[nt][e] - msafe[e >> 1]);
        ps[e >> 1] += s[nt][e];
      }
    }
    lrow[0] = lrow[0] * alpha[0] + ps[0];
    lrow[1] = lrow[1] * alpha[1] + ps[1];
#pragma unroll
    for (int dn = 0; dn < C::DN; ++dn) {
      o[dn][0] *= alpha[0];
      o[dn][1] *= alpha[0];
      o[dn][2] *= alpha[1];
      o[dn][3] *= alpha[1];
    }

#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
      const uint32_t a0 = pack_bf16x2(s[2 * kt][0], s[2 * kt][1]);
      const uint32_t a1 = pack_bf16x2(s[2 * kt][2], s[2 * kt][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      const uint32_t a3 = pack_bf16x2(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
      for (int dp = 0; dp < C::DN / 2; ++dp) {
        const int r = kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vbase + r * C::ROW_BYTES + ((c ^ (r & 7)) << 4));
        mma_bf16_16816(o[2 * dp], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_lo + gid + r * 8;
    if (row >= Lq) continue;
    const float inv = lrow[r] > 0.f ? 1.f / lrow[r] : 0.f;
    __nv_bfloat16* dst = p.out + static_cast<int64_t>(q0 + row) * p.out_stride + h * D + 2 * tig;
#pragma unroll
    for (int dn = 0; dn < C::DN; ++dn)
      *reinterpret_cast<uint32_t*>(dst + dn * 8) = pack_bf16x2(o[dn][2 * r] * inv, o[dn][2 * r + 1] * inv);
  }
}

template <class C>
static int launch_prefill_mma_t(const PrefillParams& p, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "prefill: cannot reserve %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  dim3 grid((p.max_seqlen_q + C::BM - 1) / C::BM, p.hq, p.batch);
  prefill_mma_kernel<C><<<grid, C::NW * 32, C::SMEM, stream>>>(p);
  count_launch();
  return check_launch("prefill (mma.sync) launch");
}

int launch_prefill_mma(const PrefillParams& p, cudaStream_t stream) {
  if (p.d == 128) return launch_prefill_mma_t<PrefillMmaCfg<128>>(p, stream);
  return launch_prefill_mma_t<PrefillMmaCfg<64>>(p, stream);
}

}  // namespace nvllm
