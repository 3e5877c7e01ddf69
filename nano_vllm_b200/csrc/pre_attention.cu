// Fused pre-attention step: per-head RMSNorm of q and k, NeoX-style rotary embedding of q and
// k, and the scatter of the new K/V rows into the paged cache, in one launch over the fused
// qkv activation.
//
// It stands where four launches stand in nano-vllm's Qwen3 attention block
// (nanovllm/models/qwen3.py:89-107): q_norm and k_norm (RMSNorm.rms_forward,
// nanovllm/layers/layernorm.py:17-27), rotary_emb (RotaryEmbedding.forward and
// apply_rotary_emb, nanovllm/layers/rotary_embedding.py:6-16,39-55) and store_kvcache
// (nanovllm/layers/attention.py:32-39).  Qwen2 has no q/k norm (nanovllm/models/qwen2.py:87-90):
// the weights are then NULL and only rotation and store happen.
//
// The arithmetic repeats the reference's roundings: x -> fp32, x * rsqrt(mean(x^2) + eps) rounded
// to bf16, times the bf16 weight rounded to bf16; rotation in fp32 as x1*cos - x2*sin and
// x2*cos + x1*sin with separately rounded products (no fused multiply-add), rounded to bf16.
// q and k are rewritten in place in the qkv buffer (the attention kernels read them from
// there); the rotated k row and the untouched v row are also copied to their cache slot.
//
// One warp per (token, head).  For head_dim 128 a lane owns elements {2l, 2l+1} of each half
// of the head, so the rotation partner x[i + D/2] lives in the same lane.
#include "common.cuh"

namespace nvllm {

struct PreAttnParams {
  __nv_bfloat16* qkv;
  int64_t row_stride;
  const int64_t* positions;
  const __nv_bfloat16* q_weight;  // nullable
  const __nv_bfloat16* k_weight;  // nullable
  const float* cos_sin;           // [max_position, D]: cos (D/2) then sin (D/2)
  int64_t max_position;
  float eps;
  const int32_t* slot_mapping;    // nullable: no store
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int64_t num_slots;
  int64_t n_tokens;
  int hq, hkv;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(256) pre_attention_kernel(const PreAttnParams p) {
  pdl_prologue();  // lets the attention kernel that follows get its blocks resident early
  constexpr int EPL = D / 64;  // elements per lane in each half of the head
  const int lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (unit >= p.n_tokens * heads) return;
  const int64_t tok = unit / heads;
  const int head = static_cast<int>(unit - tok * heads);
  __nv_bfloat16* row = p.qkv + tok * p.row_stride + static_cast<int64_t>(head) * D;

  int64_t slot = -1;
  if (p.slot_mapping && head >= p.hq) {
    slot = p.slot_mapping[tok];
    if (slot >= p.num_slots) {
      if (lane == 0) atomicOr(p.status, NVLLM_STATUS_BAD_SLOT);
      slot = -1;
    }
  }

  if (head >= p.hq + p.hkv) {  // a V head: copy to the cache, nothing else
    if (slot >= 0) {
      const int vh = head - p.hq - p.hkv;
      __nv_bfloat16* dst = p.v_cache + (slot * p.hkv + vh) * D;
      if constexpr (D == 128) {
        reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(row)[lane];
      } else {
        reinterpret_cast<uint32_t*>(dst)[lane] = reinterpret_cast<const uint32_t*>(row)[lane];
      }
    }
    return;
  }

  const bool is_k = head >= p.hq;
  const __nv_bfloat16* w = is_k ? p.k_weight : p.q_weight;
  float x1[EPL], x2[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    x1[e] = __bfloat162float(row[lane * EPL + e]);
    x2[e] = __bfloat162float(row[D / 2 + lane * EPL + e]);
  }
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
    const float rstd = rsqrtf(ss * (1.0f / D) + p.eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float w1 = __bfloat162float(w[lane * EPL + e]), w2 = __bfloat162float(w[D / 2 + lane * EPL + e]);
      x1[e] = __bfloat162float(__float2bfloat16(__fmul_rn(__bfloat162float(__float2bfloat16(__fmul_rn(x1[e], rstd))), w1)));
      x2[e] = __bfloat162float(__float2bfloat16(__fmul_rn(__bfloat162float(__float2bfloat16(__fmul_rn(x2[e], rstd))), w2)));
    }
  }
  int64_t pos = p.positions[tok];
  if (pos < 0 || pos >= p.max_position) pos = pos < 0 ? 0 : p.max_position - 1;
  const float* cs = p.cos_sin + pos * D;
  __nv_bfloat16 y1[EPL], y2[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const float c = cs[lane * EPL + e], s = cs[D / 2 + lane * EPL + e];
    y1[e] = __float2bfloat16(__fsub_rn(__fmul_rn(x1[e], c), __fmul_rn(x2[e], s)));
    y2[e] = __float2bfloat16(__fadd_rn(__fmul_rn(x2[e], c), __fmul_rn(x1[e], s)));
  }
  __nv_bfloat16* kdst = (is_k && slot >= 0) ? p.k_cache + (slot * p.hkv + (head - p.hq)) * D : nullptr;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    row[lane * EPL + e] = y1[e];
    row[D / 2 + lane * EPL + e] = y2[e];
    if (kdst) {
      kdst[lane * EPL + e] = y1[e];
      kdst[D / 2 + lane * EPL + e] = y2[e];
    }
  }
}

}  // namespace nvllm

extern "C" int nvllm_qk_norm_rope_store(void* qkv, int64_t row_stride, const int64_t* positions, const void* q_weight,
                                        const void* k_weight, const float* cos_sin_cache, int64_t max_position, float eps,
                                        const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t num_slots,
                                        int64_t n_tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                        void* stream) {
  using namespace nvllm;
  if (head_dim != 64 && head_dim != 128)
    return fail(NVLLM_E_GEOMETRY, "qk_norm_rope_store: head_dim=%d unsupported (64 or 128)", head_dim);
  if (num_q_heads <= 0 || num_kv_heads <= 0) return fail(NVLLM_E_GEOMETRY, "qk_norm_rope_store: head counts must be positive");
  if (n_tokens < 0 || max_position <= 0) return fail(NVLLM_E_GEOMETRY, "qk_norm_rope_store: n_tokens / max_position invalid");
  if (n_tokens == 0) return NVLLM_OK;
  if (!qkv || !positions || !cos_sin_cache) return fail(NVLLM_E_NULL, "qk_norm_rope_store: NULL pointer argument");
  if ((q_weight == nullptr) != (k_weight == nullptr))
    return fail(NVLLM_E_NULL, "qk_norm_rope_store: give both norm weights or neither");
  const int64_t width = static_cast<int64_t>(num_q_heads + 2 * num_kv_heads) * head_dim;
  if (row_stride < width) return fail(NVLLM_E_GEOMETRY, "qk_norm_rope_store: row stride smaller than (Hq+2Hkv)*D");
  if (row_stride % 8 || !aligned16(qkv)) return fail(NVLLM_E_ALIGN, "qk_norm_rope_store: qkv and its row stride must be 16-byte aligned");
  if (slot_mapping) {
    if (!k_cache || !v_cache || num_slots <= 0) return fail(NVLLM_E_NULL, "qk_norm_rope_store: slot_mapping given without caches");
    if (!aligned16(k_cache) || !aligned16(v_cache)) return fail(NVLLM_E_ALIGN, "qk_norm_rope_store: caches must be 16-byte aligned");
  }
  PreAttnParams p;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "qk_norm_rope_store: no CUDA device is usable");
  p.qkv = static_cast<__nv_bfloat16*>(qkv);
  p.row_stride = row_stride;
  p.positions = positions;
  p.q_weight = static_cast<const __nv_bfloat16*>(q_weight);
  p.k_weight = static_cast<const __nv_bfloat16*>(k_weight);
  p.cos_sin = cos_sin_cache;
  p.max_position = max_position;
  p.eps = eps;
  p.slot_mapping = slot_mapping;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.num_slots = num_slots;
  p.n_tokens = n_tokens;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  const int64_t units = n_tokens * (num_q_heads + 2 * num_kv_heads);
  const int64_t blocks = (units + 7) / 8;
  if (blocks > 0x7fffffffLL) return fail(NVLLM_E_GEOMETRY, "qk_norm_rope_store: too many tokens for one launch");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) pre_attention_kernel<128><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p);
  else pre_attention_kernel<64><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p);
  count_launch();
  return check_launch("qk_norm_rope_store launch");
}
