// Pieces shared by the tcgen05 attention kernels (forward and backward).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attn_common.cuh"
#include "tc_common.cuh"

namespace fat {
namespace tcattn {

using namespace tc;

constexpr int BLK = 128;                 // rows per query tile and keys per key tile
constexpr uint32_t kTmemCols = 512;

template <typename T> struct Pack16;
template <> struct Pack16<__nv_bfloat16> {
  static constexpr int kFmt = 1;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};
template <> struct Pack16<__half> {
  static constexpr int kFmt = 0;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// sigma(s)^4 with sigma(s) = (s/(|s|+1) + 1)/2
__device__ __forceinline__ float sigma4(float s) {
  const float sg = fmaf(s * rcp_approx(fabsf(s) + 1.0f), 0.5f, 0.5f);
  const float s2 = sg * sg;
  return s2 * s2;
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Loads one [128][D] tile (rows row0.., all of D) as D/64 boxes of 64 columns.
template <int D>
__device__ __forceinline__ void load_tile_tma(unsigned char* dst, const CUtensorMap* m, uint64_t* bar,
                                              int row0, int h, int b) {
  mbar_expect_tx(bar, BLK * D * 2);
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_4d(dst + c * (BLK * 128), m, bar, c * 64, row0, h, b);
}

}  // namespace tcattn
}  // namespace fat
