// store_kvcache: scatter the new tokens' K/V rows into the paged cache.
// Behaviour follows nanovllm/layers/attention.py:10-39 (one cache row per token, addressed
// by slot_mapping); the implementation is a 16-byte-vector copy where one thread moves one
// 16-byte piece of a K row and the matching piece of the V row.
#include "common.cuh"

namespace nvllm {

constexpr int kStoreThreads = 256;
constexpr int kStoreUnroll = 2;  // 16-byte pieces per thread per tensor

__global__ void __launch_bounds__(kStoreThreads)
store_kvcache_kernel(const uint4* __restrict__ key, int64_t key_stride16,      // row strides in 16-byte units
                     const uint4* __restrict__ value, int64_t value_stride16,
                     uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                     const int32_t* __restrict__ slot_mapping,
                     int64_t n_tokens, int pieces_per_row, int64_t num_slots, int* __restrict__ status) {
  pdl_prologue();  // lets the attention kernel that follows get its blocks resident early
  const int64_t total = n_tokens * pieces_per_row;
  const int64_t base = (static_cast<int64_t>(blockIdx.x) * kStoreThreads) * kStoreUnroll + threadIdx.x;

  uint4 kreg[kStoreUnroll], vreg[kStoreUnroll];
  int64_t dst[kStoreUnroll];
#pragma unroll
  for (int u = 0; u < kStoreUnroll; ++u) {
    const int64_t idx = base + static_cast<int64_t>(u) * kStoreThreads;
    dst[u] = -1;
    if (idx < total) {
      const int64_t tok = idx / pieces_per_row;
      const int piece = static_cast<int>(idx - tok * pieces_per_row);
      const int64_t slot = slot_mapping[tok];
      if (slot >= num_slots) {
        if (piece == 0) atomicOr(status, NVLLM_STATUS_BAD_SLOT);
      } else if (slot >= 0) {
        dst[u] = slot * pieces_per_row + piece;
        kreg[u] = __ldg(key + tok * key_stride16 + piece);
        vreg[u] = __ldg(value + tok * value_stride16 + piece);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kStoreUnroll; ++u) {
    if (dst[u] >= 0) {
      k_cache[dst[u]] = kreg[u];
      v_cache[dst[u]] = vreg[u];
    }
  }
}

}  // namespace nvllm

extern "C" int nvllm_store_kvcache(const void* key, int64_t key_row_stride,
                                   const void* value, int64_t value_row_stride,
                                   void* k_cache, void* v_cache,
                                   const int32_t* slot_mapping, int64_t n_tokens,
                                   int32_t row_elems, int64_t num_slots, void* stream) {
  using namespace nvllm;
  if (n_tokens < 0) return fail(NVLLM_E_GEOMETRY, "store_kvcache: n_tokens=%lld < 0", (long long)n_tokens);
  if (n_tokens == 0) return NVLLM_OK;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping)
    return fail(NVLLM_E_NULL, "store_kvcache: NULL pointer argument");
  if (row_elems <= 0 || row_elems % 8 != 0)
    return fail(NVLLM_E_GEOMETRY, "store_kvcache: row_elems=%d must be a positive multiple of 8", row_elems);
  if (num_slots <= 0) return fail(NVLLM_E_GEOMETRY, "store_kvcache: num_slots=%lld must be positive", (long long)num_slots);
  if (key_row_stride < row_elems || value_row_stride < row_elems)
    return fail(NVLLM_E_GEOMETRY, "store_kvcache: row strides (%lld, %lld) smaller than row_elems=%d",
                (long long)key_row_stride, (long long)value_row_stride, row_elems);
  if (key_row_stride % 8 || value_row_stride % 8)
    return fail(NVLLM_E_ALIGN, "store_kvcache: row strides (%lld, %lld) must be multiples of 8 elements",
                (long long)key_row_stride, (long long)value_row_stride);
  if (!aligned16(key) || !aligned16(value) || !aligned16(k_cache) || !aligned16(v_cache))
    return fail(NVLLM_E_ALIGN, "store_kvcache: key/value/cache pointers must be 16-byte aligned");
  int* status = status_word();
  if (!status) return fail(NVLLM_E_NO_DEVICE, "store_kvcache: no CUDA device is usable");

  const int pieces = row_elems / 8;
  const int64_t total = n_tokens * pieces;
  const int64_t per_block = static_cast<int64_t>(kStoreThreads) * kStoreUnroll;
  const int64_t blocks = (total + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) return fail(NVLLM_E_GEOMETRY, "store_kvcache: too many tokens for one launch");
  store_kvcache_kernel<<<static_cast<unsigned>(blocks), kStoreThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(key), key_row_stride / 8, static_cast<const uint4*>(value), value_row_stride / 8,
      static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache), slot_mapping, n_tokens, pieces, num_slots, status);
  count_launch();
  return check_launch("store_kvcache launch");
}
