// Host-side construction of TMA tensor maps.  The driver's encoder is looked up at run time
// through the runtime API, so the library carries no link-time dependency on libcuda.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

namespace nvllm {
namespace sm100 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool make_tmap_3d(CUtensorMap* map, const void* base, uint64_t head_dim, uint64_t heads, uint64_t rows,
                  uint64_t head_stride_elems, uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_heads) {
  EncodeTiledFn enc = encoder();
  if (!enc) {
    fail(NVLLM_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  const cuuint64_t dims[3] = {head_dim, heads, rows};
  const cuuint64_t strides[2] = {head_stride_elems * 2, row_stride_elems * 2};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {64, box_heads, box_rows};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fail(NVLLM_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu x %llu, strides %llu / %llu B)",
         (int)r, (unsigned long long)head_dim, (unsigned long long)heads, (unsigned long long)rows,
         (unsigned long long)strides[0], (unsigned long long)strides[1]);
    return false;
  }
  return true;
}

}  // namespace sm100
}  // namespace nvllm
