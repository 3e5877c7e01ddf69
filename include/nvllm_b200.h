/*
 * nvllm_b200 — C ABI of the paged-attention path for nano-vllm on NVIDIA B200 (sm_100a).
 *
 * The library replaces the three device operations behind nano-vllm's attention layer
 * (nanovllm/layers/attention.py): the Triton `store_kvcache_kernel`, the
 * `flash_attn_varlen_func` prefill call and the `flash_attn_with_kvcache` decode call.
 *
 * Conventions shared by every entry point
 *   - All tensors are bf16 (2-byte elements); metadata is int32.  Strides and extents are in
 *     ELEMENTS, never bytes.  Every data pointer and every row stride must be 16-byte aligned
 *     (8 elements); an entry point rejects anything else instead of taking a slow path.
 *   - The caller owns every buffer.  No entry point allocates, frees or synchronises, and
 *     every kernel is launched on the `stream` that is passed in (a `cudaStream_t` given as
 *     `void*`; NULL is the legacy default stream), on the device that is current.  That makes
 *     every launch legal inside CUDA stream capture.
 *   - Launch geometry depends only on host-visible arguments (batch, table width, head
 *     counts), never on device-resident lengths, so a captured graph can be replayed with
 *     new `context_lens` / `block_tables` / `slot_mapping` contents.
 *   - Return value: 0 = kernels launched; a negative NVLLM_E_* code = the arguments were
 *     rejected on the host before any launch.  `nvllm_last_error()` then holds a message.
 *     No C++ exception crosses this boundary.
 *   - Threads: one host thread per device at a time.  The first call of an entry point on a
 *     device fills small per-device caches (kernel attributes, the status word's address, the SM
 *     count) without locking; two host threads making a device's first calls at the same moment
 *     would race.  Separate processes, one per GPU, need no care.
 *   - Problems that only the device can see (a slot or block id outside the cache) never
 *     trap: the offending access is skipped and a bit is set in a device status word that
 *     `nvllm_read_status()` returns.
 *
 * KV-cache layout (nanovllm/engine/model_runner.py:136-149): one plane per layer for K and
 * one for V, each `[num_blocks, 256, Hkv, D]` contiguous.  Flat slot s = block*256 + offset;
 * element (s, h, d) sits at s*Hkv*D + h*D + d.
 */
#ifndef NVLLM_B200_H_
#define NVLLM_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define NVLLM_API __attribute__((visibility("default")))
#else
#define NVLLM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define NVLLM_BLOCK_SIZE 256 /* tokens per KV-cache block (nanovllm/engine/sequence.py:15) */

/* host-side rejection codes */
#define NVLLM_OK 0
#define NVLLM_E_NULL (-1)      /* a required pointer is NULL */
#define NVLLM_E_ALIGN (-2)     /* pointer or stride not 16-byte aligned */
#define NVLLM_E_GEOMETRY (-3)  /* unsupported head_dim / head counts / sizes */
#define NVLLM_E_WORKSPACE (-4) /* decode workspace missing or too small */
#define NVLLM_E_CUDA (-5)      /* the CUDA runtime refused the launch */
#define NVLLM_E_NO_DEVICE (-6) /* no usable sm_100 device is current */

/* bits of the device status word */
#define NVLLM_STATUS_BAD_SLOT 1  /* store_kvcache saw slot >= num_slots (row skipped) */
#define NVLLM_STATUS_BAD_BLOCK 2 /* a block_tables entry in use was outside [0,num_blocks) */
#define NVLLM_STATUS_TIMEOUT 4   /* a bounded in-kernel wait expired; that launch's output is invalid */

/*
 * Scatter the new tokens' K and V rows into the paged cache.
 * Replaces store_kvcache_kernel + store_kvcache (nanovllm/layers/attention.py:10-39):
 *   k_cache_flat[slot_mapping[i]] = key[i], same for V; a row is row_elems = Hkv*D elements.
 * key/value: [n_tokens, row_elems] with unit inner stride and the given row strides (value
 * is a strided view of the fused qkv activation in the caller).  Rows with slot < 0 are
 * skipped; rows with slot >= num_slots are skipped and flagged.  Pure copy: bit-exact.
 */
NVLLM_API int nvllm_store_kvcache(const void* key, int64_t key_row_stride,
                        const void* value, int64_t value_row_stride,
                        void* k_cache, void* v_cache,
                        const int32_t* slot_mapping, int64_t n_tokens,
                        int32_t row_elems, int64_t num_slots, void* stream);

/*
 * Paged GQA decode: one query token per sequence against context_lens[b] cached tokens.
 * Replaces the flash_attn_with_kvcache call (nanovllm/layers/attention.py:74-77).
 *   out[b,h,:] = sum_{t<ctx_b} softmax_t(scale * q[b,h].K[t,h/G]) V[t,h/G],  G = Hq/Hkv.
 * q/out: [batch, Hq, D] with unit inner strides and the given row (per sequence) strides.
 * block_tables: [batch, max_blocks] int32 with row stride bt_row_stride; only the first
 * ceil(ctx_b/256) entries of a row are read.  ctx_b == 0 gives a zero output row and
 * touches no cache memory.  One launch: the cached tokens of the whole batch are dealt out in
 * equal shares to two thread blocks per SM, whatever the individual lengths are; a sequence
 * whose tokens fall into several shares gets fp32 partial results in `workspace`, and the
 * thread block that delivers the last of them merges them (no second kernel).
 * `workspace`: nvllm_decode_workspace_bytes(...) bytes for the same (batch, Hq, Hkv, D),
 * 16-byte aligned.  Its first 64 KiB are arrival counters: ZERO-FILL THE WORKSPACE ONCE before
 * its first use; every completed call leaves the counters at zero again, so one workspace can
 * serve all later calls, of any geometry, that do not overlap on the GPU.
 * Supported: D in {64,128}; Hq % Hkv == 0; G <= 8; batch * Hkv <= 16384.
 */
NVLLM_API int nvllm_decode_paged(const void* q, int64_t q_row_stride,
                       const void* k_cache, const void* v_cache,
                       const int32_t* context_lens,
                       const int32_t* block_tables, int64_t bt_row_stride, int32_t max_blocks,
                       void* out, int64_t out_row_stride,
                       int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                       float scale, int64_t num_blocks,
                       void* workspace, int64_t workspace_bytes, void* stream);

/*
 * One decode step of the attention layer in one launch: store_kvcache of the new token of every
 * sequence followed by the paged decode, i.e. nanovllm/layers/attention.py:65-66 and :74-77
 * together.  key/value: [batch, Hkv, D] rows of the token being decoded (row strides given;
 * value may be a strided view of the fused qkv activation); slot_mapping[b] is the cache slot of
 * that token, which the model runner sets to the slot of position ctx_b - 1
 * (nanovllm/engine/model_runner.py:225-229).  The thread block that streams position ctx_b - 1
 * takes the row from key/value instead of the cache and writes it to the cache on the way, so
 * the cache ends up exactly as store_kvcache would leave it and the output is the same as
 * nvllm_store_kvcache followed by nvllm_decode_paged.  Rules that differ from the two separate
 * calls: slot_mapping[b] < 0 stores nothing (the row is read from the cache as it is); a
 * slot_mapping[b] >= 0 that is not the slot of position ctx_b - 1 is flagged
 * NVLLM_STATUS_BAD_SLOT and not stored; rows with ctx_b == 0 (the padding rows of a captured
 * batch) store nothing, where the reference scatters them to slot_mapping[b].
 * Everything else as nvllm_decode_paged (same workspace, same limits).
 */
NVLLM_API int nvllm_decode_step(const void* q, int64_t q_row_stride,
                      const void* key, int64_t key_row_stride,
                      const void* value, int64_t value_row_stride,
                      const int32_t* slot_mapping,
                      void* k_cache, void* v_cache,
                      const int32_t* context_lens,
                      const int32_t* block_tables, int64_t bt_row_stride, int32_t max_blocks,
                      void* out, int64_t out_row_stride,
                      int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                      float scale, int64_t num_blocks,
                      void* workspace, int64_t workspace_bytes, void* stream);

/* Bytes of workspace nvllm_decode_paged / nvllm_decode_step need for this geometry (0 for an
 * empty batch): the counter area plus one partial per (share, sequence) piece, sized for the
 * largest launch the library makes on any device.  Negative NVLLM_E_* on unsupported geometry.
 * Pure host arithmetic, no device needed.
 * No counterpart in the reference: flash-attn allocates its split-KV scratch internally. */
NVLLM_API int64_t nvllm_decode_workspace_bytes(int32_t batch, int32_t max_blocks,
                                     int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim);

/* How the library cuts this geometry: tokens per work unit, and the number of thread blocks a
 * launch uses on the current device (two per SM rounded down to a multiple of Hkv; the sizing
 * cap when no device is usable).  Exposed for tests and reports. */
NVLLM_API int nvllm_decode_plan(int32_t batch, int32_t max_blocks, int32_t num_q_heads,
                      int32_t num_kv_heads, int32_t head_dim,
                      int32_t* unit_tokens, int32_t* thread_blocks);

/* Size of the scratch array built into the library for nvllm_decode_paged_static. */
#define NVLLM_DECODE_STATIC_SCRATCH_BYTES (32ll << 20)

/*
 * nvllm_decode_paged for callers that cannot supply a workspace.  No counterpart in the
 * reference (flash-attn allocates its split-KV scratch through torch on every call).
 *
 * Who needs it: a host that must not, or cannot, allocate device memory once it is serving —
 * an engine that has handed every free byte of HBM to its KV cache, a latency-critical loop
 * that cannot afford the device-wide synchronisation an allocation may imply, or a thin
 * binding that only forwards pointers it received and owns no allocator.  Inputs and the
 * output are still the caller's buffers; only the split-KV partials move into the library.
 *
 * Same arguments and results as nvllm_decode_paged minus the workspace pair.  The counters and
 * partials go to a 32 MiB (NVLLM_DECODE_STATIC_SCRATCH_BYTES) array that is part of the library
 * image, so every GPU whose context loads the library carries those 32 MiB until the process
 * exits.  The call never allocates or frees anything.  Limits and rules:
 *   - a geometry whose nvllm_decode_workspace_bytes() exceeds the array is refused with
 *     NVLLM_E_WORKSPACE before anything is launched (e.g. batch 2048 with 64 query heads); use
 *     the workspace variant for those;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call outside stream capture;
 *   - all calls on a device share the one array, which still holds whatever the previous
 *     call left there.  Only the arrival counters at its head have to start at zero: they do
 *     when the library is loaded, and the thread block that merges a sequence puts its counter
 *     back to zero, so a completed call leaves them cleared.  Partials are written before they
 *     are read within one call.  Two calls whose kernels may run at the same time on one GPU
 *     (different streams, or graphs replayed concurrently) would disturb each other's counters
 *     and partials — keep calls to this entry point ordered on a device.
 */
NVLLM_API int nvllm_decode_paged_static(const void* q, int64_t q_row_stride,
                              const void* k_cache, const void* v_cache,
                              const int32_t* context_lens,
                              const int32_t* block_tables, int64_t bt_row_stride, int32_t max_blocks,
                              void* out, int64_t out_row_stride,
                              int32_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                              float scale, int64_t num_blocks, void* stream);

/*
 * Varlen causal GQA prefill.  Replaces the flash_attn_varlen_func call
 * (nanovllm/layers/attention.py:67-73).  For sequence b, query row i (0-based among its
 * Lq_b = cu_seqlens_q[b+1]-cu_seqlens_q[b] new tokens) attends keys j <= i + (Lk_b - Lq_b),
 * j over the full sequence of Lk_b = cu_seqlens_k[b+1]-cu_seqlens_k[b] tokens
 * (bottom-right aligned causal mask).  Two K/V sources:
 *   - packed (block_tables == NULL): key j of sequence b is row cu_seqlens_k[b]+j of
 *     k / v, each [total_k, Hkv, D] with the given row strides;
 *   - paged (block_tables != NULL): k / v are the cache planes and key j of sequence b is
 *     slot block_tables[b, j/256]*256 + j%256; the k/v row strides are ignored.
 * q/out: [total_q, Hq, D] with the given row strides.  Lq_b == 0 is legal (no work).
 * total_q / total_k are the row counts of q and of packed k/v (ignored for k/v in paged
 * mode); they bound the tiled loads, nothing past them is read.
 * Cache contents past a sequence's length are never observed (stale NaN/Inf cannot leak).
 * Supported: D in {64,128}; Hq % Hkv == 0; batch <= 1024 (nano-vllm schedules at most 512
 * sequences per step); more is rejected with NVLLM_E_GEOMETRY.  Runs on the persistent tcgen05
 * kernel.  The environment variable NVLLM_PREFILL_IMPL=mma, read on every call, selects a
 * warp-level mma.sync kernel instead (cross-check for tests and A/B baseline for measurements).
 */
NVLLM_API int nvllm_prefill_varlen(const void* q, int64_t q_row_stride,
                         const void* k, int64_t k_row_stride,
                         const void* v, int64_t v_row_stride,
                         const int32_t* block_tables, int64_t bt_row_stride, int32_t max_blocks,
                         void* out, int64_t out_row_stride,
                         const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                         int64_t total_q, int64_t total_k,
                         int32_t batch, int32_t max_seqlen_q, int32_t max_seqlen_k,
                         int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                         float scale, int64_t num_blocks, void* stream);

/*
 * Fused pre-attention step over the fused qkv activation [n_tokens, (Hq + 2*Hkv) * D] (bf16,
 * row stride given): per-head RMSNorm of q and k (skipped when both weights are NULL), NeoX
 * rotary embedding of q and k from a [max_position, D] fp32 table (cos half, then sin half),
 * in place; then the rotated k rows and the v rows are copied to their cache slots (skipped
 * when slot_mapping is NULL; slot < 0 rows are skipped).  positions is int64 [n_tokens].
 * Replaces, in nano-vllm's attention blocks (nanovllm/models/qwen3.py:89-107,
 * qwen2.py:87-90): RMSNorm.rms_forward x2 (nanovllm/layers/layernorm.py:17-27),
 * RotaryEmbedding.forward (nanovllm/layers/rotary_embedding.py:39-55) and store_kvcache
 * (nanovllm/layers/attention.py:32-39), with the same intermediate roundings.
 * Supported: D in {64,128}.
 */
NVLLM_API int nvllm_qk_norm_rope_store(void* qkv, int64_t row_stride, const int64_t* positions,
                             const void* q_weight, const void* k_weight,
                             const float* cos_sin_cache, int64_t max_position, float eps,
                             const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t num_slots,
                             int64_t n_tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                             void* stream);

/*
 * Token sampling in one pass over the logits [batch, vocab] (bf16, or fp32 when logits_are_fp32
 * != 0; row stride in elements): tokens[b] = argmax_i(logits[b,i]) when temperatures[b] == 0,
 * else a draw from softmax(logits[b] / temperatures[b]) made as
 *     argmax_i( logits[b,i] / T_b - ln(e_i + 1e-10) ),   e_i ~ Exponential(1),
 * which is the reference's argmax(softmax(logits / T) / (e + 1e-10)) without the normaliser.
 * Replaces Sampler.forward (nanovllm/layers/sampler.py:10-26).  exponential_noise, when not
 * NULL, is the caller's [batch, vocab] fp32 draw of e (then the result is the reference's token
 * for the same draw); when NULL, e comes from a Philox4x32-10 generator keyed by `seed` and
 * counted by (row, position, `step`): stateless, the same (seed, step) gives the same tokens,
 * and the caller advances `step` once per call.  tokens is int64 [batch].  Ties go to the lowest
 * index; NaN logits are never chosen.  Rows that start on a 16-byte boundary are read with
 * 16-byte loads, others element by element (no alignment is required).
 */
NVLLM_API int nvllm_sample_tokens(const void* logits, int32_t logits_are_fp32, int64_t row_stride,
                        const float* temperatures, const float* exponential_noise, int64_t noise_row_stride,
                        uint64_t seed, uint64_t step, int64_t* tokens, int32_t batch, int32_t vocab,
                        void* stream);

/*
 * The same pass for tensor-parallel ranks that each hold the logits of one slice of the
 * vocabulary [vocab_offset, vocab_offset + vocab): instead of a token, row b yields
 * candidates[b], one int64 that packs the slice's best (score, global index) so that a signed MAX
 * over the ranks' candidates selects the token nvllm_sample_tokens would select from the
 * concatenated row (same seed and step on every rank; the generated noise depends on the global
 * index only).  nvllm_sample_unpack turns merged candidates into token ids.  Together with an
 * 8-byte-per-row MAX reduction they stand where ParallelLMHead.forward gathers every rank's
 * [batch, vocab / ranks] logits on rank 0 and concatenates them
 * (nanovllm/layers/embed_head.py:78-87) before Sampler.forward (nanovllm/layers/sampler.py:10-26).
 */
NVLLM_API int nvllm_sample_candidates(const void* logits, int32_t logits_are_fp32, int64_t row_stride,
                            const float* temperatures, const float* exponential_noise, int64_t noise_row_stride,
                            uint64_t seed, uint64_t step, int64_t vocab_offset, int64_t* candidates,
                            int32_t batch, int32_t vocab, void* stream);
NVLLM_API int nvllm_sample_unpack(const int64_t* candidates, int64_t* tokens, int32_t batch, void* stream);

/*
 * Decode-step inputs for a captured CUDA graph, in one launch.  `staged` is a device copy of
 * one host staging block holding, at the given BYTE offsets: tokens int64[batch] (last token of
 * each sequence), lens int32[batch] (sequence lengths, the new token included), offsets
 * int32[batch+1] and the concatenated block tables int32[offsets[batch]].  The kernel fills rows
 * [0, graph_batch) of the graph's static tensors: input_ids / positions (int64), slot_mapping /
 * context_lens (int32) and block_tables (int32, table_width columns, row stride in elements):
 * rows < batch from the staged data (slot = last block * 256 + position of the newest token in
 * it; table padded with -1 up to used_width = the widest table of the batch, 0 beyond), rows >=
 * batch all zero.  Replaces the per-step copies of ModelRunner.prepare_decode /
 * prepare_block_tables (nanovllm/engine/model_runner.py:151-159, 218-249) and the clear-and-copy
 * of the graph buffers in run_model (model_runner.py:271-282), with bit-identical buffers over
 * the rows the graph reads.
 */
NVLLM_API int nvllm_decode_step_inputs(const void* staged, int64_t tokens_off, int64_t lens_off, int64_t offsets_off,
                             int64_t blocks_off, int32_t batch, int32_t graph_batch, int32_t used_width,
                             int32_t table_width, int64_t* input_ids, int64_t* positions,
                             int32_t* slot_mapping, int32_t* context_lens, int32_t* block_tables,
                             int64_t bt_row_stride, void* stream);

/*
 * All-reduce (sum, bf16) over peer memory for tensor-parallel ranks on one node, one process per
 * GPU.  Replaces dist.all_reduce in RowParallelLinear.forward (nanovllm/layers/linear.py:195-199)
 * for tensors up to `max_bytes`.  Set-up, once per process and device, outside stream capture:
 *   nvllm_ar_init(rank, world, max_bytes, handle_out)  allocates this rank's flag + staging area
 *       (8 KB + 8 * max_bytes of device memory) and writes its CUDA IPC handle
 *       (nvllm_ar_handle_bytes() bytes) to handle_out;
 *   the caller gathers the handles of all ranks (rank order) by its own means;
 *   nvllm_ar_connect(all_handles)  maps every peer's area.
 * nvllm_ar_allreduce(in, out, n_elems, stream) then launches one kernel; every rank must make the
 * same sequence of calls with the same n_elems, and a rank's calls must execute one after the
 * other (one stream, or otherwise serialised: the staging buffers belong to one call at a
 * time).  in == out is allowed; both 16-byte aligned;
 * n_elems * 2 <= max_bytes.  All ranks get bit-identical sums (fp32 accumulation in rank order).
 * The call picks one of four protocols from (n_elems, world, max_bytes) alone, the same on every
 * rank: (1) flagged 16-byte cells pushed to every peer (small tensors: one NVLink crossing of
 * latency, twice the bytes on the wire); (4) flagged cells in two shots at more than two ranks (a
 * rank sends the cells of slice j to its owner j only, the owner sums and sends the result cells to
 * everyone); (2) staging + flags with every rank pulling all peers' tensors (one shot); (3)
 * staging + flags in two shots (pushed reduce-scatter + all-gather).  nvllm_ar_protocol() reports
 * the choice; nvllm_ar_set_protocol() forces one where it applies (0 = automatic; measurement aid;
 * every rank must set the same).
 * No allocation, synchronisation or host read in the call: legal during stream capture, and a
 * captured graph can be replayed (call counts live in device memory).  A peer that does not
 * arrive within ~1 s of SM clocks sets NVLLM_STATUS_TIMEOUT; that call's output is invalid and
 * later calls no longer wait.  nvllm_ar_shutdown() unmaps and frees (synchronises the device).
 */
NVLLM_API int64_t nvllm_ar_handle_bytes(void);
NVLLM_API int nvllm_ar_init(int32_t rank, int32_t world, int64_t max_bytes, void* handle_out);
NVLLM_API int nvllm_ar_connect(const void* all_handles);
NVLLM_API int64_t nvllm_ar_max_bytes(void); /* 0 until connected */
/* How long a rank waits for its peers before it gives up (default ~1000 ms of SM clocks).  Ranks
 * that run loosely coupled (one may be seconds behind while it compiles or captures) need more. */
NVLLM_API int nvllm_ar_set_wait_ms(int64_t ms);
NVLLM_API int nvllm_ar_allreduce(const void* in, void* out, int64_t n_elems, void* stream);
NVLLM_API int nvllm_ar_set_protocol(int32_t protocol);
/* Pure host arithmetic; no device needed. */
NVLLM_API int nvllm_ar_protocol(int64_t n_elems, int32_t world, int64_t max_bytes, int32_t forced);
NVLLM_API int nvllm_ar_shutdown(void);
/* The same hand-shake and arithmetic with all `world` ranks emulated by ONE cooperative launch on
 * the current device (inputs[r], outputs[r]: rank r's tensors; scratch: zero-filled before the
 * first call, nvllm_ar_emulated_scratch_bytes(world, max_bytes) bytes, kept between calls).  For
 * testing the protocol where fewer GPUs than ranks are at hand; absent_rank >= 0 makes that rank
 * stay away, so that the others' bounded waits run out (~1 s) and report NVLLM_STATUS_TIMEOUT
 * without any fault; -1 = all present.  protocol: as nvllm_ar_set_protocol.  No counterpart in
 * the reference. */
NVLLM_API int64_t nvllm_ar_emulated_scratch_bytes(int32_t world, int64_t max_bytes);
NVLLM_API int nvllm_ar_allreduce_emulated(int32_t world, const void* const* inputs, void* const* outputs,
                                int64_t n_elems, void* scratch, int64_t scratch_bytes, int64_t max_bytes,
                                int32_t absent_rank, int32_t protocol, void* stream);

/* Row-parallel projection fused with its all-reduce: out[m, n] = sum over ranks of x_r[m, k] w_r[n, k]^T,
 * bf16 in and out.  Replaces F.linear followed by dist.all_reduce in RowParallelLinear.forward
 * (nanovllm/layers/linear.py:195-199) for bias-free projections of decode-sized batches: ONE launch
 * per rank computes the rank's partial on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM)
 * and its epilogue sums the partials over peer memory tile by tile -- each rank's fp32 partial is
 * rounded to bf16 (as F.linear would have), a tile's partials go to the tile's owner rank as
 * flagged cells, the owner adds them in rank order in fp32, rounds once and sends the result to
 * every rank (two shots), or -- at two ranks and for small outputs -- go to every rank, which adds
 * them in rank order itself (one shot); either way all ranks hold the same bits.  Needs nvllm_ar_init + nvllm_ar_connect; every rank
 * makes the same calls in the same order, and calls may be mixed freely with nvllm_ar_allreduce.
 * x, weight, out: 16-byte aligned, row strides (elements) multiples of 8; k a multiple of 8, n of 32.
 * nvllm_ar_gemm_tile() returns the tile width (32, 64 or 128) the call would use, or 0 when the
 * shape does not fit the cell areas (4 * n * 128 * ceil(m / 128) bytes needed out of max_bytes; 2, 4
 * or 8 ranks); such shapes are refused with NVLLM_E_GEOMETRY (use the unfused pair).
 * Pure host arithmetic; no device needed. */
NVLLM_API int nvllm_ar_gemm_tile(int64_t m, int64_t n, int64_t k, int32_t world, int64_t max_bytes);
NVLLM_API int nvllm_ar_gemm_allreduce(const void* x, int64_t x_stride, const void* weight, int64_t w_stride, void* out,
                            int64_t out_stride, int64_t m, int64_t n, int64_t k, void* stream);
/* The same with all ranks emulated by ONE cooperative launch on the current device (xs[r] [m, k],
 * weights[r] [n, k], outputs[r] [m, n], all contiguous; scratch as for nvllm_ar_allreduce_emulated).
 * mode: 0 = the kernel's own choice between one and two shots, 1 = one shot where the cell areas
 * hold it, 2 = two shots.  No counterpart in the reference. */
NVLLM_API int nvllm_ar_gemm_allreduce_emulated(int32_t world, const void* const* xs, const void* const* weights,
                                     void* const* outputs, int64_t m, int64_t n, int64_t k, void* scratch,
                                     int64_t scratch_bytes, int64_t max_bytes, int32_t mode, void* stream);

/* Known-answer check of the tensor-core building blocks the prefill kernel is made of
 * (TMA swizzled loads, shared-memory and instruction descriptors, TMEM loads and stores):
 * out_ss = A B^T and out_ts = A B for A, B [128,128] bf16 row-major, outputs [128,128] fp32.
 * A diagnostic for new driver / toolkit versions.  No counterpart in the reference. */
NVLLM_API int nvllm_selftest_umma(const void* a, const void* b, float* out_ss, float* out_ts, void* stream);

/* Failure-detection check that faults nothing: a one-block kernel waits on a barrier that
 * nothing signals.  The wait gives up after about one second, a second waiter leaves through
 * the block's abort flag, NVLLM_STATUS_TIMEOUT is recorded in the status word, and the block
 * frees its tensor memory and ends normally (the context stays usable).  device_result (two
 * int32 in device memory) receives 0/0: both waits reported failure.  No counterpart in the
 * reference. */
NVLLM_API int nvllm_selftest_wait_expiry(int32_t* device_result, void* stream);

/* Message for the last negative return value on this thread ("" if none).
 * No counterpart in the reference (it raises Python exceptions). */
NVLLM_API const char* nvllm_last_error(void);

/* Copies the current device's status word to *host_out and clears it.  Synchronises the
 * device: call it between steps, never during stream capture.  Returns 0 or NVLLM_E_*.
 * No counterpart in the reference. */
NVLLM_API int nvllm_read_status(int32_t* host_out);

/* ABI version of this header (bumped on any signature change). */
NVLLM_API int nvllm_abi_version(void);

/* How many kernels this library has launched in this process (all entry points, all
 * devices).  Monotonic; used by the benchmark to report its launch count. */
NVLLM_API int64_t nvllm_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NVLLM_B200_H_ */
