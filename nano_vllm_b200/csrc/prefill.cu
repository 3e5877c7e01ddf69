// nvllm_prefill_varlen: argument checks and kernel selection.
#include <cstdlib>

#include "common.cuh"
#include "prefill.cuh"

extern "C" int nvllm_prefill_varlen(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                    const void* v, int64_t v_row_stride, const int32_t* block_tables,
                                    int64_t bt_row_stride, int32_t max_blocks, void* out, int64_t out_row_stride,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int64_t total_q,
                                    int64_t total_k, int32_t batch, int32_t max_seqlen_q, int32_t max_seqlen_k, int32_t num_q_heads,
                                    int32_t num_kv_heads, int32_t head_dim, float scale, int64_t num_blocks,
                                    void* stream) {
  using namespace nvllm;
  if (head_dim != 64 && head_dim != 128)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: head_dim=%d unsupported (64 or 128)", head_dim);
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: Hq=%d must be a positive multiple of Hkv=%d", num_q_heads, num_kv_heads);
  if (batch < 0 || num_q_heads > 65535)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: batch=%d / Hq=%d outside the launch limits", batch, num_q_heads);
  if (max_seqlen_q < 0 || max_seqlen_k < 0)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: negative max_seqlen");
  if (total_q < 0 || total_k < 0) return fail(NVLLM_E_GEOMETRY, "prefill_varlen: negative total_q / total_k");
  if (batch == 0 || max_seqlen_q == 0 || total_q == 0) return NVLLM_OK;
  if (!q || !k || !v || !out || !cu_seqlens_q || !cu_seqlens_k)
    return fail(NVLLM_E_NULL, "prefill_varlen: NULL pointer argument");
  const int64_t qrow = static_cast<int64_t>(num_q_heads) * head_dim;
  const int64_t kvrow = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (q_row_stride < qrow || out_row_stride < qrow)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: q/out row stride smaller than Hq*D");
  if (q_row_stride % 8 || out_row_stride % 8 || !aligned16(q) || !aligned16(out) || !aligned16(k) || !aligned16(v))
    return fail(NVLLM_E_ALIGN, "prefill_varlen: pointers and row strides must be 16-byte aligned");
  if (block_tables) {
    if (max_blocks <= 0 || bt_row_stride < max_blocks || num_blocks <= 0)
      return fail(NVLLM_E_GEOMETRY, "prefill_varlen: paged mode needs max_blocks>0, bt_row_stride>=max_blocks, num_blocks>0");
  } else {
    if (k_row_stride < kvrow || v_row_stride < kvrow)
      return fail(NVLLM_E_GEOMETRY, "prefill_varlen: k/v row stride smaller than Hkv*D");
    if (k_row_stride % 8 || v_row_stride % 8)
      return fail(NVLLM_E_ALIGN, "prefill_varlen: k/v row strides must be multiples of 8 elements");
  }
  // The persistent tcgen05 kernel is the product.  NVLLM_PREFILL_IMPL=mma (read on every call)
  // selects the warp-level mma.sync kernel instead: the cross-check of the tests and the A/B
  // baseline of measurements, never chosen by the library itself.
  const char* forced = std::getenv("NVLLM_PREFILL_IMPL");
  const bool has_rows = block_tables || total_k > 0;
  const bool use_mma = (forced && forced[0] == 'm') || !has_rows;
  if (!use_mma && batch > kPrefillMaxBatch)
    return fail(NVLLM_E_GEOMETRY, "prefill_varlen: batch=%d exceeds the %d sequences of one launch", batch, kPrefillMaxBatch);
  if (batch > 65535) return fail(NVLLM_E_GEOMETRY, "prefill_varlen: batch=%d outside the launch limits", batch);
  PrefillParams p;
  p.status = status_word();
  if (!p.status) return fail(NVLLM_E_NO_DEVICE, "prefill_varlen: no CUDA device is usable");
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_row_stride;
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.k_stride = k_row_stride;
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.v_stride = v_row_stride;
  p.block_tables = block_tables;
  p.bt_stride = bt_row_stride;
  p.max_blocks = max_blocks;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_row_stride;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.batch = batch;
  p.max_seqlen_q = max_seqlen_q;
  p.max_seqlen_k = max_seqlen_k;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.g = num_q_heads / num_kv_heads;
  p.d = head_dim;
  p.pack = 1;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.num_blocks = num_blocks;
  if (use_mma) return launch_prefill_mma(p, static_cast<cudaStream_t>(stream));
  return launch_prefill_tcp(p, total_q, total_k, static_cast<cudaStream_t>(stream));
}
