// Tile geometry, barrier roles and the bounded wait shared by the tcgen05 prefill kernels.
#pragma once

#include "common.cuh"
#include "sm100.cuh"

namespace nvllm {

namespace tc {
constexpr int BM = 128, BN = 64, D = 128, KST = 2;
constexpr int Q_BYTES = BM * D * 2;        // 32 KB: two [128 x 64] swizzled sub-tiles
constexpr int Q_SUB = Q_BYTES / 2;
constexpr int KV_BYTES = BN * D * 2;       // 16 KB: two [64 x 64] swizzled sub-tiles
constexpr int KV_SUB = KV_BYTES / 2;
constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + KST * KV_BYTES, OFF_BAR = OFF_V + KST * KV_BYTES;
constexpr int SMEM = OFF_BAR + 256 + 1024;  // + barriers + alignment slack
constexpr int TMEM_COLS = 256;              // S/P buffers: [0,64) and [64,128); O: [128,256)
constexpr int NTHREADS = 192;
constexpr float kRescaleThreshold = 8.f;    // log2 units
// One tcgen05.commit per MMA group: a commit that follows a group of a different kind costs the
// tensor pipe a bubble (~100-200 cycles measured), so each completion is signalled once and
// shared by all its waiters.  QK_DONE[s]: S buffer s holds S_j (softmax) and K stage s is free
// (producer).  PV_DONE[s]: V stage s is free (producer), O includes tile j (rescale, epilogue).
enum Bar {
  Q_FULL = 0, K_FULL0, K_FULL1, V_FULL0, V_FULL1, QK_DONE0, QK_DONE1, PV_DONE0, PV_DONE1,
  P_FULL0, P_FULL1, DRAIN, NUM_BARS
};
// self-test tile geometry (128 x 128 operands)
constexpr int TILE_BYTES = 128 * 128 * 2, SUB_BYTES = TILE_BYTES / 2;
}  // namespace tc

// Three-input max and packed two-lane fp32 arithmetic (sm_100): they halve the issue slots of the
// row-maximum, scale-and-subtract and row-sum passes of the softmax.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Bounded wait that also gives up as soon as another role has aborted.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (sm100::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (sm100::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > sm100::kWaitLimitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

}  // namespace nvllm
