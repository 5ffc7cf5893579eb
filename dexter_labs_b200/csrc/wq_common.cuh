// Shared pieces of the weight-only quantised GEMM kernels for sm_100a: tile and
// ring constants, the bit-pattern dequantisation arithmetic, the barrier slots of
// the warp-specialised pipeline, and the host helpers that encode TMA tensor maps.
#pragma once
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/dexter_b200.h"
#include "sm100_ptx.cuh"

namespace dx {
// ------------------------------------------------------------------ constants
constexpr int kTileN = 128;      // weight columns per tile (UMMA M)
constexpr int kUnitRows = 64;    // packed rows per plane of a unit (one plane = 64 logical k)
constexpr int kQBytes = kTileN * kUnitRows;  // 8192: bytes of 64 packed rows of a tile
constexpr int kWStage = kQBytes;
constexpr int kMaxWStages = 16;  // packed-weight ring; always a multiple of kAStages
constexpr int kAStages = 4;      // dequantised-tile ring in TMEM
constexpr int kACol0 = 256;      // TMEM column where that ring starts
constexpr int kThreads = 768;    // 24 warps
constexpr int kDequantThreads = 128;  // one team
constexpr int kTeamWarps = kDequantThreads / 32;
constexpr int kEpilogueThreads = 128;
constexpr int kSmemBudget = 227 * 1024 - 4096;
constexpr int kMaxTiles = 16384;  // tile counters reserved in every workspace

// -------------------------------------------------------------- dequant math
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float hi, float lo) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// Two nibbles (bits 0..3 and 16..19 of `w`) -> two bf16 weights.  OR-ing a nibble
// into the mantissa of 0x4300 gives 128 + q exactly; `zero2` holds 128 + zero
// point in both halves (0x4308 = 136.0 for the symmetric midpoint 8), so the
// subtract is exact and the multiply is the only rounding.
__device__ __forceinline__ uint32_t deq4(uint32_t w, uint32_t zero2, uint32_t scale2) {
  const uint32_t v = (w & 0x000F000Fu) | 0x43004300u;
  return mul_bf16x2(sub_bf16x2(v, zero2), scale2);
}
// One byte -> fp32 by bit pattern: 0x4B0000qq = 8388608 + q.  `cz` = 8388608 +
// zero point; subtract and multiply are both exact in fp32 (8-bit x 8-bit
// significands), so the later cvt.rn to bf16 is the only rounding.
__device__ __forceinline__ float deq8(uint32_t word, uint32_t byte_sel, float cz, float scale) {
  const float f = __uint_as_float(prmt(word, 0x4B000000u, 0x7650u + byte_sel));
  return (f - cz) * scale;
}
__device__ __forceinline__ uint32_t dup_lo(uint32_t w) { return prmt(w, w, 0x1010u); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t w) { return prmt(w, w, 0x3232u); }
__device__ __forceinline__ float bf16lo_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// First unit of CTA c and the CTA that owns unit u, for `total` units cut into
// `ctas` contiguous ranges.
__host__ __device__ inline long long range_begin(long long c, long long total, long long ctas) {
  return c * total / ctas;
}
__host__ __device__ inline int owner_of(long long u, long long total, long long ctas) {
  return static_cast<int>(((u + 1) * ctas - 1) / total);
}

// ----------------------------------------------------------------- the kernel
// Barrier slots in shared memory.
// ready[t]: unit slot t has its activations in shared memory (TMA bytes) AND its
// dequantised weights in TMEM (128 arrivals of one team); free[t]: the MMAs that
// read slot t are done (one tcgen05.commit), so both may be overwritten.
constexpr int kBarFullW = 0, kBarEmptyW = 16, kBarReady = 32, kBarFree = 36, kBarAccFull = 40,
              kBarAccEmpty = 42, kNumBars = 44;

__device__ __forceinline__ uint32_t bar_count(int i) {
  if (i < kBarEmptyW) return 1;                    // full_w: producer's expect_tx
  // One arrival per WARP, not per thread: 128 arrivals on one barrier word serialise in
  // the shared-memory atomic unit and put ~500 cycles on every hand-over.
  if (i < kBarReady) return kTeamWarps;            // empty_w: the four warps of one team
  if (i < kBarFree) return kTeamWarps + 1;         // ready: team warps + activation producer
  if (i < kBarAccEmpty) return 1;                  // free, acc_full: one tcgen05.commit
  return kEpilogueThreads / 32;                    // acc_empty: the four epilogue warps
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// rank-2 or rank-3 tiled map; dims/box innermost first, strides in bytes for dims 1..rank-1.
inline bool make_map(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int rank,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t d[3], st[2];
  cuuint32_t bx[3], es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  return fn(m, dt, rank, const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct DeviceInfo {
  int sms = 0;
  bool attr_set = false;
};
inline DeviceInfo& device_info() {
  static std::mutex mu;
  static std::unordered_map<int, DeviceInfo> infos;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = infos[dev];
  if (d.sms == 0) cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
  return d;
}

// Shapes the tensor-core kernel takes.  Everything else goes to wq_gemm_simt.
inline bool tc_supported(int M, int N, int K, int group, int bits) {
  if (M < 1) return false;
  if (N % 16 || N < 16) return false;
  const int rows = bits == 4 ? K / 2 : K;
  if (bits == 4 && (K % 2)) return false;
  if (rows % kUnitRows) return false;
  if (group % kUnitRows || K % group) return false;
  if (K / group < 1) return false;
  // tiles = column tiles x token blocks of 128
  if (static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + 127) / 128) > kMaxTiles) return false;
  return true;
}

constexpr size_t kStatusBytes = 256;

// Polls (of about a quarter of a microsecond) a wait on a flag written by ANOTHER GPU makes
// before it gives up; set through dxb_set_wait_limit_ms, about a second by default.
unsigned wait_tries();

}  // namespace dx
