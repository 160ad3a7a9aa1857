// Tile formats and register-level tile math shared by the streaming linear kernel and the persistent decode kernel.
#pragma once
#include "common.cuh"

namespace pt {

template <int WFMT> struct WTraits;
template <> struct WTraits<PT_W_INT4> { static constexpr int kChunkK = 128, kUnits = 4, kTileBytes = 1056; };
template <> struct WTraits<PT_W_FP8> { static constexpr int kChunkK = 64, kUnits = 2, kTileBytes = 1024; };
template <> struct WTraits<PT_W_FP16> { static constexpr int kChunkK = 32, kUnits = 1, kTileBytes = 1024; };

static inline int chunk_k(int wfmt) { return wfmt == PT_W_INT4 ? 128 : (wfmt == PT_W_FP8 ? 64 : 32); }
static inline int tile_bytes(int wfmt) { return wfmt == PT_W_INT4 ? 1056 : 1024; }
static inline int row_bytes(int wfmt, int k) { return wfmt == PT_W_INT4 ? k / 2 : (wfmt == PT_W_FP8 ? k : 2 * k); }

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t two_bytes) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xFFFFu), __NV_E4M3);
  return (uint32_t)r.x | ((uint32_t)r.y << 16);
}
constexpr float kOffA = 1032.0f, kOffB = 72.0f;  // 1024 + 8 and 64 + 8

// One 32-bit-word group (8 consecutive k) of one row -> the four half2 fragment registers (k0,k1) (k2,k3) (k4,k5) (k6,k7).
// INT4: registers 0 and 2 carry the offset 1032, 1 and 3 the offset 72 (removed after the mma).
template <int WFMT> __device__ __forceinline__ void expand8(const uint4 &v, int u, uint32_t (&f)[4]) {
  const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
  if constexpr (WFMT == PT_W_INT4) {
    const uint32_t w = wd[u], w8 = w >> 8;
    f[0] = (w & 0x000F000Fu) | 0x64006400u;
    f[1] = (w & 0x00F000F0u) | 0x54005400u;
    f[2] = (w8 & 0x000F000Fu) | 0x64006400u;
    f[3] = (w8 & 0x00F000F0u) | 0x54005400u;
  } else if constexpr (WFMT == PT_W_FP8) {
    f[0] = cvt_e4m3x2(wd[2 * u]);
    f[1] = cvt_e4m3x2(wd[2 * u] >> 16);
    f[2] = cvt_e4m3x2(wd[2 * u + 1]);
    f[3] = cvt_e4m3x2(wd[2 * u + 1] >> 16);
  } else {
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
}


}  // namespace pt
