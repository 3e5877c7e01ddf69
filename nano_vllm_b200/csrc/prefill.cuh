// Parameters shared by the prefill kernels and their host-side dispatcher.
#pragma once
#include "common.cuh"

namespace nvllm {

struct PrefillParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  const __nv_bfloat16* k;  // packed K rows, or the K cache plane when block_tables != nullptr
  int64_t k_stride;
  const __nv_bfloat16* v;
  int64_t v_stride;
  const int32_t* block_tables;  // nullptr = packed K/V
  int64_t bt_stride;
  int max_blocks;
  __nv_bfloat16* out;
  int64_t out_stride;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int batch, max_seqlen_q, max_seqlen_k;
  int hq, hkv, g, d;
  int pack;  // persistent tcgen05 kernel only: query heads packed into one tile (1..8)
  float scale_log2e;
  int64_t num_blocks;
  int* status;
};

// Sequences per launch of the persistent kernel (its per-sequence tables live in shared memory).
// The engine schedules at most 512 sequences per step (nanovllm/config.py:10).
constexpr int kPrefillMaxBatch = 1024;

// Warp-level mma.sync kernel: every supported geometry; cross-check and A/B baseline only
// (batch <= 65535).
int launch_prefill_mma(const PrefillParams& p, cudaStream_t stream);
// tcgen05 / TMEM / TMA kernel in persistent blocks that pull (sequence, query tile, head) items
// from a global counter; batch <= kPrefillMaxBatch.  total_q / total_k bound the tiled loads.
int launch_prefill_tcp(const PrefillParams& p, int64_t total_q, int64_t total_k, cudaStream_t stream);

}  // namespace nvllm
