// Shared device helpers: element-type traits, 16-byte vector pack/unpack, the rational
// sigmoid pieces, warp/group reductions, and the host-side error plumbing of the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fat_b200.h"

namespace fat {

// Streaming multiprocessors of the current device (cudaDevAttrMultiProcessorCount, cached per device; 148 on a
// B200: 2 dies x 74).  Grids of the grid-stride kernels are sized in multiples of it.
int num_sms();

// ---------------------------------------------------------------- host-side errors
void set_error(const char* fmt, ...);          // defined in cabi.cu (thread-local buffer)
int  check_launch(const char* what);           // cudaGetLastError -> FAT_ERR_LAUNCH

// ---------------------------------------------------------------- element traits
template <typename T> struct Elem;
template <> struct Elem<float> {
  using C = float;                              // compute type
  static __device__ __forceinline__ float to_c(float v) { return v; }
  static __device__ __forceinline__ float from_c(float v) { return v; }
};
template <> struct Elem<double> {
  using C = double;
  static __device__ __forceinline__ double to_c(double v) { return v; }
  static __device__ __forceinline__ double from_c(double v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  using C = float;
  static __device__ __forceinline__ float to_c(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_c(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  using C = float;
  static __device__ __forceinline__ float to_c(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_c(float v) { return __float2half_rn(v); }
};

// A "pack" is W consecutive elements moved with one memory instruction.  W*sizeof(T) is
// 16 bytes on the fast paths and sizeof(T) (W = 1) on the unaligned / ragged fallback.
template <typename T, int W>
__device__ __forceinline__ void load_pack(const T* p, typename Elem<T>::C (&out)[W]) {
  if constexpr (W * sizeof(T) == 16) {
    uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));      // streaming: read once
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < W; ++i) out[i] = Elem<T>::to_c(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) out[i] = Elem<T>::to_c(p[i]);
  }
}

template <typename T, int W>
__device__ __forceinline__ void load_pack_cached(const T* p, typename Elem<T>::C (&out)[W]) {
  if constexpr (W * sizeof(T) == 16) {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < W; ++i) out[i] = Elem<T>::to_c(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) out[i] = Elem<T>::to_c(p[i]);
  }
}

template <typename T, int W>
__device__ __forceinline__ void store_pack(T* p, const typename Elem<T>::C (&in)[W]) {
  if constexpr (W * sizeof(T) == 16) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < W; ++i) e[i] = Elem<T>::from_c(in[i]);
    __stcs(reinterpret_cast<uint4*>(p), raw);                    // streaming: written once
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) p[i] = Elem<T>::from_c(in[i]);
  }
}

// ---------------------------------------------------------------- rational pieces
// r = 1/(|x|+1).  fp32 uses the special-function reciprocal (about 1 ulp), one instruction instead of
// the correctly rounded sequence: these kernels are bandwidth-bound only as long as the arithmetic stays
// light, and 1 ulp is two orders of magnitude inside the float32 bar.
__device__ __forceinline__ float  rcp1p_abs(float x)  {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fabsf(x) + 1.0f));
  return r;
}
__device__ __forceinline__ double rcp1p_abs(double x) { return 1.0 / (fabs(x) + 1.0); }

// sigma(x) = (x r + 1)/2
template <typename C> __device__ __forceinline__ C rsigmoid(C x, C r) { return (x * r + C(1)) * C(0.5); }

template <typename C> __device__ __forceinline__ C sgn(C x) { return C((x > C(0)) - (x < C(0))); }

// ---------------------------------------------------------------- reductions
template <typename C>
__device__ __forceinline__ C warp_sum(C v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace fat
