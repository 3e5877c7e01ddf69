// Shared by the peer-memory all-reduce (allreduce.cu) and the GEMM whose epilogue does the same
// sum (gemm_allreduce.cu): layout of a rank's peer-mapped area, the flagged-cell helpers, and the
// per-device host state.
#pragma once

#include "common.cuh"
#include "sm100.cuh"

namespace nvllm {
namespace ar {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 128;
constexpr int kThreads = 512;
constexpr int64_t kFlagBytes = kMaxBlocks * kMaxRanks * 4;
constexpr int64_t kEpochOff = kFlagBytes;                      // u32[kMaxBlocks]
constexpr int64_t kBrokenOff = kEpochOff + kMaxBlocks * 4;     // u32 latch
constexpr int64_t kCellEpochOff = kBrokenOff + 64;             // u32[kMaxBlocks], call counts of the cell protocol
constexpr int64_t kHeaderBytes = 8192;
static_assert(kCellEpochOff + kMaxBlocks * 4 <= kHeaderBytes, "header");
// Every call uses the same grid, whatever the size: the blocks' call counts then advance in
// lock-step, so all blocks of a call use the same staging buffer and the two-buffer argument
// holds for the whole tensor (a block with no work still counts the call).
constexpr int kGrid = 128;
constexpr int kEmulatedGrid = 16;  // x ranks blocks must be resident together on one device
static_assert(kGrid <= kMaxBlocks, "flag slots");
constexpr int kAreas = 8;  // staging 0/1, cells 0/1, result 0/1, result cells 0/1: max_bytes each
enum Protocol { kAuto = 0, kCells = 1, kOneShot = 2, kTwoShot = 3, kCellsTwoShot = 4 };
// At more than two ranks, cells to every peer put 2 x bytes x (w-1) on a rank's wire, cells in two
// shots 4 x bytes x (w-1)/w but cost one more NVLink crossing and a second round of waiting.  The
// first wins up to this size (measured: 512 KiB 10.8 against 12.3 us at 4 ranks, 17.7 against 21.2 at
// 8; 1 MiB 15.7 against 13.6 at 4 ranks and too large for the cell areas at 8).
constexpr int64_t kCellsOneShotMaxBytes = 512 << 10;

struct Peers {
  unsigned char* base[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_volatile16(uint4* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void add4(float (&acc)[4], uint32_t lo, uint32_t hi) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi));
  acc[0] += a.x;
  acc[1] += a.y;
  acc[2] += b.x;
  acc[3] += b.y;
}
__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// ---- host state (one per device of this process) ---------------------------------------------
struct State {
  bool ready = false, connected = false;
  int rank = 0, world = 0;
  int force = kAuto;
  int64_t stage_bytes = 0;
  long long wait_cycles = sm100::kWaitLimitCycles;
  unsigned char* own = nullptr;
  Peers peers{};
};
// State of the current device (nullptr when no device is usable).
State* current_state();

}  // namespace ar
}  // namespace nvllm
