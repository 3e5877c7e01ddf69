// Diagnostics of the tcgen05 / TMEM / TMA building blocks that the prefill kernel is made of:
// a known-answer test of the descriptors (SS form with K-major operands, TS form with an
// MN-major shared-memory operand), and a bounded-wait check that lets a wait run out on purpose
// without faulting anything.
#include <cstdlib>

#include "common.cuh"
#include "prefill.cuh"
#include "sm100.cuh"
#include "prefill_tc.cuh"

namespace nvllm {
using namespace sm100;

// ---- known-answer check of the building blocks --------------------------------------------
// out1 = A B^T   (SS form: A and B both K-major tiles in shared memory)
// out2 = A B     (TS form: A as packed bf16 in TMEM, B as an MN-major shared-memory tile)
// A, B: [128,128] bf16 row-major; out1, out2: [128,128] fp32.
__global__ void __launch_bounds__(160, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __nv_bfloat16* __restrict__ a, float* __restrict__ out1, float* __restrict__ out2,
                     int* __restrict__ status) {
  using namespace tc;
  extern __shared__ unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + 2 * TILE_BYTES;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + 2 * TILE_BYTES + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + 2 * TILE_BYTES + 72);
  if (tid == 0) {
    mbar_init(bar(0), 1);    // tiles landed
    mbar_init(bar(1), 1);    // SS product done
    mbar_init(bar(2), 128);  // P written
    mbar_init(bar(3), 1);    // TS product done
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t A = base, B = base + TILE_BYTES;

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), 2 * TILE_BYTES);
      tma_load_3d(A, &tmap_a, bar(0), 0, 0, 0);
      tma_load_3d(A + SUB_BYTES, &tmap_a, bar(0), 64, 0, 0);
      tma_load_3d(B, &tmap_b, bar(0), 0, 0, 0);
      tma_load_3d(B + SUB_BYTES, &tmap_b, bar(0), 64, 0, 0);
      bool ok = wait_or_abort(bar(0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t koff = (ks >> 2) * SUB_BYTES + (ks & 3) * 32;
          umma_ss(tmem, umma_desc(A + koff, 16, 1024), umma_desc(B + koff, 16, 1024), umma_idesc(128, 128, 0, 0), ks > 0);
        }
        umma_commit(bar(1));
        ok = wait_or_abort(bar(2), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + 128, tmem + ks * 8, umma_desc(B + ks * 2048, SUB_BYTES, 1024), umma_idesc(128, 128, 0, 1), ks > 0);
        umma_commit(bar(3));
      }
    }
  } else {
    const int r = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    bool ok = wait_or_abort(bar(1), 0, abort_flag);
    tc_fence_after();
    if (ok) {
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_addr + c * 32, v);
        tmem_wait_ld();
        for (int e = 0; e < 32; ++e) out1[r * 128 + c * 32 + e] = __uint_as_float(v[e]);
      }
      // stage row r of A as packed bf16 pairs in TMEM columns [0,64)
      uint32_t pk[64];
      const uint32_t* arow = reinterpret_cast<const uint32_t*>(a + r * 128);
      for (int c = 0; c < 64; ++c) pk[c] = arow[c];
      tmem_st32(tmem + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st32(tmem + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(2));
      ok = wait_or_abort(bar(3), 0, abort_flag);
      tc_fence_after();
      if (ok) {
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem + 128 + lane_addr + c * 32, v);
          tmem_wait_ld();
          for (int e = 0; e < 32; ++e) out2[r * 128 + c * 32 + e] = __uint_as_float(v[e]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(status, NVLLM_STATUS_TIMEOUT);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---- bounded-wait check ---------------------------------------------------------------------
// One block allocates TMEM, then a thread waits on an mbarrier that nothing ever arrives at.
// The wait must run out (about a second), set the abort flag that the other roles poll, record
// NVLLM_STATUS_TIMEOUT, and the block must still free its TMEM and end normally.
__global__ void __launch_bounds__(64, 1) wait_expiry_selftest_kernel(int* __restrict__ status, int* __restrict__ result) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 64);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  bool ok = true;
  if (tid == 0) ok = wait_or_abort(smem_u32(&bars[0]), 0, abort_flag);   // runs out on the clock
  if (tid == 32) ok = wait_or_abort(smem_u32(&bars[1]), 0, abort_flag);  // leaves early through the abort flag
  if (tid == 0) result[0] = ok ? 1 : 0;
  if (tid == 32) result[1] = ok ? 1 : 0;
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(status, NVLLM_STATUS_TIMEOUT);
  if (warp == 1) tmem_dealloc(tmem_slot, 64);
}

// ---- host side ---------------------------------------------------------------------------

template <class K>
static int opt_in_smem(K kernel, int bytes, bool* done, const char* what) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || done[dev]) return NVLLM_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(NVLLM_E_CUDA, "%s: cannot reserve %d bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  done[dev] = true;
  return NVLLM_OK;
}


}  // namespace nvllm

extern "C" int nvllm_selftest_wait_expiry(int32_t* device_result, void* stream) {
  using namespace nvllm;
  if (!device_result) return fail(NVLLM_E_NULL, "selftest_wait_expiry: device_result is NULL");
  int* status = status_word();
  if (!status) return fail(NVLLM_E_NO_DEVICE, "selftest_wait_expiry: no CUDA device is usable");
  wait_expiry_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, device_result);
  count_launch();
  return check_launch("selftest_wait_expiry launch");
}

extern "C" int nvllm_selftest_umma(const void* a, const void* b, float* out_ss, float* out_ts, void* stream) {
  using namespace nvllm;
  if (!a || !b || !out_ss || !out_ts) return fail(NVLLM_E_NULL, "selftest_umma: NULL pointer argument");
  if (!aligned16(a) || !aligned16(b)) return fail(NVLLM_E_ALIGN, "selftest_umma: inputs must be 16-byte aligned");
  int* status = status_word();
  if (!status) return fail(NVLLM_E_NO_DEVICE, "selftest_umma: no CUDA device is usable");
  static bool attr_done[64] = {false};
  const int smem = 2 * tc::TILE_BYTES + 128 + 1024;
  int rc = opt_in_smem(umma_selftest_kernel, smem, attr_done, "selftest_umma");
  if (rc) return rc;
  CUtensorMap ma, mb;
  if (!sm100::make_tmap_3d(&ma, a, 128, 1, 128, 128, 128, 128)) return NVLLM_E_CUDA;
  if (!sm100::make_tmap_3d(&mb, b, 128, 1, 128, 128, 128, 128)) return NVLLM_E_CUDA;
  umma_selftest_kernel<<<1, 160, smem, static_cast<cudaStream_t>(stream)>>>(
      ma, mb, static_cast<const __nv_bfloat16*>(a), out_ss, out_ts, status);
  count_launch();
  return check_launch("selftest_umma launch");
}
