// Token sampling in one pass over the logits.
//
// Stands where nano-vllm's Sampler.forward stands (nanovllm/layers/sampler.py:10-26), which
// spends eight elementwise / reduction launches over a [batch, vocab] fp32 copy of the logits:
//   greedy = argmax(logits);  probs = softmax(logits / T);
//   sample = argmax(probs / (Exponential(1) + 1e-10));  token = (T == 0) ? greedy : sample.
// argmax(p_i / e_i) is the Gumbel-max ("exponential race") way of drawing from p.  Since the
// softmax normaliser and the row maximum are common to a row, the same token is
//   argmax_i ( logit_i / T  -  ln(e_i + 1e-10) ),
// which needs neither the maximum nor the sum: one read of the row, no intermediate tensor.
//
// Two noise sources.  (1) `noise` given: e_i is read from the caller's [batch, vocab] fp32
// tensor; with the tensor the reference drew, the result is the reference's token (up to
// rounding when two candidates tie to ~1e-6 relative).  (2) `noise` NULL: e_i = -ln(1 - v)
// with v uniform in (0,1) from a Philox4x32-10 counter-based generator keyed by (seed) and
// counted by (row, position in the row, step); no state is kept between calls, the same
// (seed, step) reproduces the same tokens.
//
// A row is read by one thread-block cluster of 1, 2, 4 or 8 blocks of 256 threads (the fewer
// the rows, the more blocks each gets, so that a decode batch of any size spreads over the 148
// SMs); 16-byte loads, four in flight per thread.  Each block reduces to one candidate, block 0
// of the cluster collects the others' candidates from their shared memory.  Ties go to the
// lowest index.
//
// Tensor parallelism: nano-vllm's LM head leaves every rank with the logits of its own slice of
// the vocabulary and then gathers all slices on rank 0 and concatenates them
// (nanovllm/layers/embed_head.py:78-87) before it samples.  The candidate form of this kernel
// makes that traffic unnecessary: every rank reduces its slice to one (score, global index)
// candidate per row, packed into an int64 whose signed order is "higher score first, then lower
// index"; a MAX over the ranks (8 bytes per row) then picks the token that the one-rank kernel
// would have picked from the concatenated row, because the noise is generated from the global
// index.  nvllm_sample_unpack turns the winning candidates into token ids.
#include <cooperative_groups.h>

#include "common.cuh"

namespace nvllm {

struct SampleParams {
  const void* logits;
  int64_t row_stride;
  const float* temperatures;
  const float* noise;  // nullable
  int64_t noise_stride;
  uint64_t seed, step;
  int64_t* tokens;          // token ids, or packed candidates when `candidates` is set
  int vocab;                // elements in a row of `logits`
  int64_t offset;           // global vocabulary index of element 0 of a row
  int candidates;
};

// (score, index) as one int64 that orders like "higher score, then lower index".
__device__ __forceinline__ long long pack_candidate(float score, int idx) {
  int s = __float_as_int(score);
  s = s >= 0 ? s : s ^ 0x7fffffff;  // order-preserving map of float bits to a signed integer
  return (static_cast<long long>(s) << 32) | static_cast<long long>(0xffffffffu - static_cast<unsigned int>(idx));
}

// Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// ln of an Exponential(1) draw made from 32 random bits.  v = (bits + 0.5) / 2^32 is uniform in
// (0,1) and e = -ln(1 - v); for small v the series keeps the relative precision that 1 - v
// would lose (small e decides which unlikely token wins, large e never matters).
__device__ __forceinline__ float ln_exponential(uint32_t bits) {
  const float v = (static_cast<float>(bits >> 8) + 0.5f) * 5.9604644775390625e-08f;  // 24 bits, never 0 or 1
  float e;
  if (v < 0.03125f) {
    // the low 8 bits refine v where it is small enough for them to matter
    const float vf = (static_cast<float>(bits) + 0.5f) * 2.3283064365386963e-10f;
    e = vf * (1.f + vf * (0.5f + vf * (0.33333334f + vf * 0.25f)));
  } else {
    e = -__logf(1.f - v);
  }
  return __logf(e);
}

struct Best {
  float score;
  int idx;
};
__device__ __forceinline__ void take(Best& b, float s, int i) {
  // NaN never wins; ties keep the lower index
  if (s > b.score || (s == b.score && i < b.idx)) {
    b.score = s;
    b.idx = i;
  }
}
// Same for a thread's own elements, which it visits in rising index order.
__device__ __forceinline__ void take_next(Best& b, float s, int i) {
  if (s > b.score) {
    b.score = s;
    b.idx = i;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

// Build-time shape (measurement aid): resident blocks per SM the register budget is held to, and
// 16-byte loads in flight per thread.
#ifndef NVLLM_SAMPLER_MINBLOCKS
#define NVLLM_SAMPLER_MINBLOCKS 4
#endif
#ifndef NVLLM_SAMPLER_UNROLL
#define NVLLM_SAMPLER_UNROLL 4
#endif

template <typename T>
__global__ void __launch_bounds__(256, NVLLM_SAMPLER_MINBLOCKS) sample_kernel(const SampleParams p) {
  constexpr int VEC = 16 / sizeof(T);  // elements per 16-byte load: 8 bf16 or 4 fp32
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int csize = static_cast<int>(cluster.num_blocks()), crank = static_cast<int>(cluster.block_rank());
  const int row = blockIdx.x / csize;
  const int tid = crank * blockDim.x + threadIdx.x;  // thread index within the row's cluster
  const int nthreads = csize * blockDim.x;
  const T* x = static_cast<const T*>(p.logits) + static_cast<int64_t>(row) * p.row_stride;
  const float* nz = p.noise ? p.noise + static_cast<int64_t>(row) * p.noise_stride : nullptr;
  const float t = p.temperatures[row];
  const bool greedy = !(t > 0.f) && !(t < 0.f);  // T == 0 (or NaN): plain argmax, as torch.where(T == 0, ...)
  const float inv_t = greedy ? 1.f : 1.f / t;
  const uint2 key = make_uint2(static_cast<uint32_t>(p.seed), static_cast<uint32_t>(p.seed >> 32));

  Best best{-INFINITY, 0x7fffffff};
  // score of element i given its logit; `bits` only used by the generator path
  auto score_of = [&](float logit, int i, uint32_t bits) {
    float s = logit * inv_t;
    if (!greedy) s -= nz ? __logf(nz[i] + 1e-10f) : ln_exponential(bits);
    return s;
  };

  // 16-byte loads need an aligned row, and a slice that starts on a group of four positions
  // (one Philox call covers four consecutive global positions)
  const int off = static_cast<int>(p.offset);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (off & 3) == 0;
  const int n_vec = vec_ok ? p.vocab / VEC : 0;
  auto consume = [&](const uint4& raw, int v) {
    const T* e = reinterpret_cast<const T*>(&raw);
    uint32_t bits[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (!greedy && !nz) {
#pragma unroll
      for (int h = 0; h < VEC / 4; ++h) {
        // counter: (group of 4 positions, row, step lo, step hi) -- unique per element and call
        const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>((off >> 2) + v * (VEC / 4) + h), static_cast<uint32_t>(row),
                                                 static_cast<uint32_t>(p.step), static_cast<uint32_t>(p.step >> 32)),
                                      key);
        bits[4 * h] = r.x; bits[4 * h + 1] = r.y; bits[4 * h + 2] = r.z; bits[4 * h + 3] = r.w;
      }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) take_next(best, score_of(to_f32<T>(e[k]), v * VEC + k, bits[k]), off + v * VEC + k);
  };
  // four 16-byte loads in flight per thread before any of them is used
  constexpr int UNROLL = NVLLM_SAMPLER_UNROLL;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  int v = tid;
  for (; v + (UNROLL - 1) * nthreads < n_vec; v += UNROLL * nthreads) {
    uint4 raw[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) raw[u] = xv[v + u * nthreads];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) consume(raw[u], v + u * nthreads);
  }
  for (; v < n_vec; v += nthreads) consume(xv[v], v);
  // tail (and whole rows that are not 16-byte aligned): one element at a time, same counters
  for (int i = n_vec * VEC + tid; i < p.vocab; i += nthreads) {
    uint32_t b = 0;
    if (!greedy && !nz) {
      const int gi = off + i;  // global position
      const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(gi >> 2), static_cast<uint32_t>(row),
                                               static_cast<uint32_t>(p.step), static_cast<uint32_t>(p.step >> 32)),
                                    key);
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      b = w[gi & 3];
    }
    take_next(best, score_of(to_f32<T>(x[i]), i, b), off + i);
  }

  // block argmax: shuffle inside a warp, shared memory across the warps; then across the cluster
  auto warp_reduce = [&]() {
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
      const float s = __shfl_xor_sync(0xffffffffu, best.score, sh);
      const int i = __shfl_xor_sync(0xffffffffu, best.idx, sh);
      take(best, s, i);
    }
  };
  warp_reduce();
  __shared__ float w_score[8];
  __shared__ int w_idx[8];
  __shared__ float blk_score;
  __shared__ int blk_idx;
  const int lt = threadIdx.x;
  if ((lt & 31) == 0) {
    w_score[lt >> 5] = best.score;
    w_idx[lt >> 5] = best.idx;
  }
  __syncthreads();
  if (lt < 32) {
    const int nw = (blockDim.x + 31) >> 5;
    best.score = lt < nw ? w_score[lt] : -INFINITY;
    best.idx = lt < nw ? w_idx[lt] : 0x7fffffff;
    warp_reduce();
    if (lt == 0) {
      blk_score = best.score;
      blk_idx = best.idx;
    }
  }
  cluster.sync();  // every block's candidate is in its shared memory
  if (crank == 0 && lt < 32) {
    best.score = -INFINITY;
    best.idx = 0x7fffffff;
    if (lt < csize) {
      best.score = *cluster.map_shared_rank(&blk_score, lt);
      best.idx = *cluster.map_shared_rank(&blk_idx, lt);
    }
    warp_reduce();
    // a row of NaN / -inf only: token 0, like an argmax over equal values (after the merge, for
    // candidates: the sentinel index loses against any real candidate of another rank)
    if (lt == 0) {
      if (p.candidates) p.tokens[row] = pack_candidate(best.score, best.idx);
      else p.tokens[row] = best.idx == 0x7fffffff ? 0 : best.idx;
    }
  }
  cluster.sync();  // no block leaves while its shared memory may still be read
}

__global__ void sample_unpack_kernel(const long long* packed, int64_t* tokens, int batch) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const unsigned int idx = 0xffffffffu - static_cast<unsigned int>(packed[b] & 0xffffffffll);
  tokens[b] = idx == 0x7fffffffu ? 0 : static_cast<int64_t>(idx);
}

static int sample_launch(const void* logits, int32_t logits_are_fp32, int64_t row_stride, const float* temperatures,
                         const float* exponential_noise, int64_t noise_row_stride, uint64_t seed, uint64_t step,
                         int64_t vocab_offset, int candidates, int64_t* tokens, int32_t batch, int32_t vocab, void* stream);

}  // namespace nvllm

extern "C" int nvllm_sample_tokens(const void* logits, int32_t logits_are_fp32, int64_t row_stride,
                                   const float* temperatures, const float* exponential_noise, int64_t noise_row_stride,
                                   uint64_t seed, uint64_t step, int64_t* tokens, int32_t batch, int32_t vocab,
                                   void* stream) {
  return nvllm::sample_launch(logits, logits_are_fp32, row_stride, temperatures, exponential_noise, noise_row_stride, seed, step,
                              0, 0, tokens, batch, vocab, stream);
}

extern "C" int nvllm_sample_candidates(const void* logits, int32_t logits_are_fp32, int64_t row_stride,
                                       const float* temperatures, const float* exponential_noise, int64_t noise_row_stride,
                                       uint64_t seed, uint64_t step, int64_t vocab_offset, int64_t* candidates, int32_t batch,
                                       int32_t vocab, void* stream) {
  using namespace nvllm;
  if (vocab_offset < 0 || vocab_offset + vocab > 0x7ffffffell)
    return fail(NVLLM_E_GEOMETRY, "sample_candidates: vocab_offset=%lld invalid", (long long)vocab_offset);
  return sample_launch(logits, logits_are_fp32, row_stride, temperatures, exponential_noise, noise_row_stride, seed, step,
                       vocab_offset, 1, candidates, batch, vocab, stream);
}

extern "C" int nvllm_sample_unpack(const int64_t* candidates, int64_t* tokens, int32_t batch, void* stream) {
  using namespace nvllm;
  if (batch < 0) return fail(NVLLM_E_GEOMETRY, "sample_unpack: batch=%d invalid", batch);
  if (batch == 0) return NVLLM_OK;
  if (!candidates || !tokens) return fail(NVLLM_E_NULL, "sample_unpack: NULL pointer argument");
  if (reinterpret_cast<uintptr_t>(candidates) % 8 || reinterpret_cast<uintptr_t>(tokens) % 8)
    return fail(NVLLM_E_ALIGN, "sample_unpack: pointers must be 8-byte aligned");
  sample_unpack_kernel<<<(batch + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(candidates), tokens, batch);
  count_launch();
  return check_launch("sample_unpack launch");
}

namespace nvllm {
static int sample_launch(const void* logits, int32_t logits_are_fp32, int64_t row_stride, const float* temperatures,
                         const float* exponential_noise, int64_t noise_row_stride, uint64_t seed, uint64_t step,
                         int64_t vocab_offset, int candidates, int64_t* tokens, int32_t batch, int32_t vocab, void* stream) {
  if (batch < 0 || vocab <= 0) return fail(NVLLM_E_GEOMETRY, "sample_tokens: batch=%d vocab=%d invalid", batch, vocab);
  if (batch == 0) return NVLLM_OK;
  if (!logits || !temperatures || !tokens) return fail(NVLLM_E_NULL, "sample_tokens: NULL pointer argument");
  if (row_stride < vocab || (exponential_noise && noise_row_stride < vocab))
    return fail(NVLLM_E_GEOMETRY, "sample_tokens: a row stride is smaller than vocab");
  const size_t esz = logits_are_fp32 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(logits) % esz || reinterpret_cast<uintptr_t>(tokens) % 8 ||
      reinterpret_cast<uintptr_t>(temperatures) % 4 || reinterpret_cast<uintptr_t>(exponential_noise) % 4)
    return fail(NVLLM_E_ALIGN, "sample_tokens: a pointer is not aligned to its element size");
  SampleParams p;
  p.logits = logits;
  p.row_stride = row_stride;
  p.temperatures = temperatures;
  p.noise = exponential_noise;
  p.noise_stride = noise_row_stride;
  p.seed = seed;
  p.step = step;
  p.tokens = tokens;
  p.vocab = vocab;
  p.offset = vocab_offset;
  p.candidates = candidates;
  // rows whose start is not 16-byte aligned take the element-wise path inside the kernel.
  // Blocks per row: as many (1, 2, 4, 8) as keep the grid within one resident wave of
  // 8 blocks on every SM of this device, and no more than the row has work for.
  const int sms = num_sms();
  if (sms <= 0) return fail(NVLLM_E_NO_DEVICE, "sample_tokens: no CUDA device is usable");
  int csize = 8;
  while (csize > 1 && (static_cast<int64_t>(batch) * csize > static_cast<int64_t>(sms) * (NVLLM_SAMPLER_MINBLOCKS > 4 ? NVLLM_SAMPLER_MINBLOCKS : 8) || vocab < csize * 256 * 8)) csize >>= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(batch) * csize, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = logits_are_fp32 ? cudaLaunchKernelEx(&cfg, sample_kernel<float>, p)
                                  : cudaLaunchKernelEx(&cfg, sample_kernel<__nv_bfloat16>, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(NVLLM_E_CUDA, "sample_tokens launch: %s", cudaGetErrorString(e));
  }
  count_launch();
  return check_launch("sample_tokens launch");
}
}  // namespace nvllm
