// Decode-step inputs written into a CUDA graph's static buffers by one launch.
//
// nano-vllm prepares a decode step with six small host->device copies
// (ModelRunner.prepare_decode, prepare_block_tables, prepare_sample:
// nanovllm/engine/model_runner.py:151-159, 218-258) and then, to replay a captured graph, clears
// the graph's five static input tensors and copies the fresh ones into their first rows
// (run_model, model_runner.py:271-282): about sixteen launches and copies before the graph can
// start.  Here the host packs the step into ONE staging block (one copy) and this kernel expands
// it into the static buffers, rows [0, graph_bs):
//   row r <  bs: input_ids = last token, positions = context_lens = sequence length,
//                slot_mapping = last block * 256 + offset of the newest token,
//                block_tables = the sequence's blocks, -1 up to the widest table of the batch,
//                0 beyond it (what clearing the buffer and copying a [bs, widest] table leaves);
//   row r >= bs: all zero (the padding rows of a graph captured for a larger batch).
// The results are bit-identical to the reference's buffers over the rows the graph reads.
#include "common.cuh"

namespace nvllm {

struct DecodeInputsParams {
  const int64_t* tokens;    // [bs]
  const int32_t* lens;      // [bs]
  const int32_t* offsets;   // [bs + 1] into flat_blocks
  const int32_t* flat_blocks;
  int bs, graph_bs, used_width, table_width;
  int64_t* input_ids;
  int64_t* positions;
  int32_t* slot_mapping;
  int32_t* context_lens;
  int32_t* block_tables;
  int64_t bt_stride;
};

__global__ void __launch_bounds__(64) decode_inputs_kernel(const DecodeInputsParams p) {
  const int r = blockIdx.x;
  int32_t* bt = p.block_tables + static_cast<int64_t>(r) * p.bt_stride;
  if (r >= p.bs) {
    if (threadIdx.x == 0) {
      p.input_ids[r] = 0;
      p.positions[r] = 0;
      p.slot_mapping[r] = 0;
      p.context_lens[r] = 0;
    }
    for (int j = threadIdx.x; j < p.table_width; j += blockDim.x) bt[j] = 0;
    return;
  }
  const int len = p.lens[r];
  const int o0 = p.offsets[r], n = p.offsets[r + 1] - o0;
  if (threadIdx.x == 0) {
    p.input_ids[r] = p.tokens[r];
    p.positions[r] = len;
    p.context_lens[r] = len;
    // Sequence.last_block_num_tokens (nanovllm/engine/sequence.py:58-63) and block_table[-1]
    const int num_blocks = (len + kBlockSize - 1) / kBlockSize;
    const int last = n > 0 ? p.flat_blocks[o0 + n - 1] : 0;
    p.slot_mapping[r] = last * kBlockSize + (len - (num_blocks - 1) * kBlockSize) - 1;
  }
  for (int j = threadIdx.x; j < p.table_width; j += blockDim.x)
    bt[j] = j < n ? p.flat_blocks[o0 + j] : (j < p.used_width ? -1 : 0);
}

}  // namespace nvllm

extern "C" int nvllm_decode_step_inputs(const void* staged, int64_t tokens_off, int64_t lens_off, int64_t offsets_off,
                                        int64_t blocks_off, int32_t batch, int32_t graph_batch, int32_t used_width,
                                        int32_t table_width, int64_t* input_ids, int64_t* positions,
                                        int32_t* slot_mapping, int32_t* context_lens, int32_t* block_tables,
                                        int64_t bt_row_stride, void* stream) {
  using namespace nvllm;
  if (batch < 0 || graph_batch < batch || table_width <= 0 || used_width < 0 || used_width > table_width)
    return fail(NVLLM_E_GEOMETRY, "decode_step_inputs: batch=%d graph_batch=%d used_width=%d table_width=%d invalid", batch,
                graph_batch, used_width, table_width);
  if (graph_batch == 0) return NVLLM_OK;
  if (!staged || !input_ids || !positions || !slot_mapping || !context_lens || !block_tables)
    return fail(NVLLM_E_NULL, "decode_step_inputs: NULL pointer argument");
  if (bt_row_stride < table_width) return fail(NVLLM_E_GEOMETRY, "decode_step_inputs: table row stride smaller than its width");
  const uintptr_t base = reinterpret_cast<uintptr_t>(staged);
  if ((base + tokens_off) % 8 || (base + lens_off) % 4 || (base + offsets_off) % 4 || (base + blocks_off) % 4 ||
      tokens_off < 0 || lens_off < 0 || offsets_off < 0 || blocks_off < 0)
    return fail(NVLLM_E_ALIGN, "decode_step_inputs: a section of the staging block is misaligned");
  DecodeInputsParams p;
  const char* b = static_cast<const char*>(staged);
  p.tokens = reinterpret_cast<const int64_t*>(b + tokens_off);
  p.lens = reinterpret_cast<const int32_t*>(b + lens_off);
  p.offsets = reinterpret_cast<const int32_t*>(b + offsets_off);
  p.flat_blocks = reinterpret_cast<const int32_t*>(b + blocks_off);
  p.bs = batch;
  p.graph_bs = graph_batch;
  p.used_width = used_width;
  p.table_width = table_width;
  p.input_ids = input_ids;
  p.positions = positions;
  p.slot_mapping = slot_mapping;
  p.context_lens = context_lens;
  p.block_tables = block_tables;
  p.bt_stride = bt_row_stride;
  decode_inputs_kernel<<<graph_batch, 64, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launch();
  return check_launch("decode_step_inputs launch");
}
