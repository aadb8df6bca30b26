// Rational attention of ONE new token per sequence over a key/value cache: the step `generate` repeats.
//
// The reference's generate() (algebraic_model.py:239-265) runs the whole model over the whole prefix for every new
// token.  With causal attention and a relative (ALiBi) bias the keys and values of earlier positions never change, so
// a cache of them turns the attention of a decode step into
//     out = sum_j f_j v_j / (sum_j f_j + eps),   f_j = sigma(q . k_j * scale - slope * (n - j))^4,   j = 0..n
// for the single query at position n: no running maximum, so partial sums over key ranges simply add.  The step is
// bound by reading the cache once (2 * (n+1) * D elements per (batch, head)).
//
// One launch appends the new key/value row to the cache and attends over it.  A (batch, head) pair is served by a
// thread-block cluster of 1-8 CTAs that split the key range; the partial sums meet in the first CTA through
// distributed shared memory (one fixed summation order: the result is bit-reproducible).  Within a CTA a key row is
// spread over D/W lanes (W = elements per 16-byte pack), every lane keeps its slice of q and of the accumulator in
// registers, and each thread has the cache rows of kStages - 1 steps (kUnroll key rows and value rows each) in flight
// through a shared-memory ring while it sums one step.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "../../include/fat_b200.h"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace fat {
namespace {

#ifndef FAT_DEC_THREADS
#define FAT_DEC_THREADS 128
#endif
#ifndef FAT_DEC_UNROLL
#define FAT_DEC_UNROLL 4
#endif
#ifndef FAT_DEC_STAGES
#define FAT_DEC_STAGES 3          // steps whose cache rows are in flight or in use at once, per CTA
#endif
#ifndef FAT_DEC_FILL
#define FAT_DEC_FILL 3            // the key range of a (batch, head) pair is split until there are this many CTAs per SM
#endif
#ifndef FAT_DEC_MIN_ROWS
#define FAT_DEC_MIN_ROWS 256      // ... but no CTA gets fewer rows of a full cache than this (more, smaller clusters measured slower)
#endif
#ifndef FAT_DEC_MINB
#define FAT_DEC_MINB 4            // CTAs per SM the register budget is cut for
#endif
constexpr int kDecThreads = FAT_DEC_THREADS;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kUnroll = FAT_DEC_UNROLL;
constexpr int kStages = FAT_DEC_STAGES;
constexpr int kRingBytes = kStages * kUnroll * 2 * kDecThreads * 16;

struct DecodeParams {
  const void* q; const void* k_new; const void* v_new;     // [B,H,D], strides {batch, head}
  void* k_cache; void* v_cache;                             // [B,H,capacity,D], strides {batch, head, token}
  const int* n_cached;                                      // [B]: rows already in the cache; the new row goes there
  const float* slopes; void* out;                           // out [B,H,D], strides {batch, head}
  int B, H, capacity;
  int64_t qs[2], kns[2], vns[2], os[2], kcs[3], vcs[3];
  float scale, eps;
  int* status;
};

template <typename T, int W>
__device__ __forceinline__ void unpack(const uint4& raw, float (&f)[W]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < W; ++i) f[i] = Elem<T>::to_c(e[i]);
}

// Two neighbouring float32 values as one 64-bit register pair: fma.rn.f32x2 works on both at once.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }

// A 16-byte pack as W/2 float32 pairs.
template <typename T> struct Pairs;
template <> struct Pairs<__nv_bfloat16> {
  static __device__ __forceinline__ void get(const uint4& raw, f32x2 (&o)[4]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = pk2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
};
template <> struct Pairs<__half> {
  static __device__ __forceinline__ void get(const uint4& raw, f32x2 (&o)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); o[i] = pk2(f.x, f.y); }
  }
};
template <> struct Pairs<float> {
  static __device__ __forceinline__ void get(const uint4& raw, f32x2 (&o)[2]) {
    o[0] = pk2(__uint_as_float(raw.x), __uint_as_float(raw.y));
    o[1] = pk2(__uint_as_float(raw.z), __uint_as_float(raw.w));
  }
};

template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads, FAT_DEC_MINB)
attn_decode_kernel(const DecodeParams p) {
  constexpr int W = 16 / sizeof(T);            // elements per pack
  constexpr int LPR = D / W;                   // lanes per key row
  constexpr int RPW = 32 / LPR;                // key rows a warp handles at once
  constexpr int kStep = kDecWarps * RPW;       // key rows a CTA handles at once
  static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "head size must spread over a power-of-two lane count");
  __shared__ float red[kDecWarps][D + 1];
  __shared__ float tot[D + 1];

  cg::cluster_group cluster = cg::this_cluster();
  const int n_split = int(cluster.num_blocks()), split = int(cluster.block_rank());
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane / LPR, c = lane % LPR;

  int n = p.n_cached[b];
  if (n < 0 || n >= p.capacity) {              // no room for the new row: report it, touch nothing, give zeros
    if (tid == 0 && split == 0 && p.status) atomicOr(p.status, int(FAT_DEV_CACHE_FULL));
    n = -1;
  }
  const int total = n + 1;
  const int per = ((total + n_split - 1) / n_split + kStep - 1) / kStep * kStep;
  const int lo = split * per, hi = min(total, lo + per);

  T* kc = static_cast<T*>(p.k_cache) + b * p.kcs[0] + h * p.kcs[1];
  T* vc = static_cast<T*>(p.v_cache) + b * p.vcs[0] + h * p.vcs[1];
  if (n >= 0 && n >= lo && n < hi && tid < 2 * LPR) {           // the CTA that owns row n appends it first
    const bool is_v = tid >= LPR;
    const int cc = tid % LPR;
    const T* src = is_v ? static_cast<const T*>(p.v_new) + b * p.vns[0] + h * p.vns[1]
                        : static_cast<const T*>(p.k_new) + b * p.kns[0] + h * p.kns[1];
    T* dst = (is_v ? vc + n * p.vcs[2] : kc + n * p.kcs[2]);
    reinterpret_cast<uint4*>(dst)[cc] = __ldg(reinterpret_cast<const uint4*>(src) + cc);
  }
  __syncthreads();                             // the row is read back below by threads of this CTA only

  static_assert(kUnroll == 4 && LPR >= 4, "the four-row transpose reduction below needs four rows and four lanes per row");
  constexpr int P = W / 2;                     // float32 pairs per pack
  f32x2 q2[P];
  {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1]) + c);
    float qf[W];
    unpack<T, W>(raw, qf);
#pragma unroll
    for (int i = 0; i < P; ++i) q2[i] = pk2(qf[2 * i] * p.scale, qf[2 * i + 1] * p.scale);
  }
  const float slope = p.slopes[h];
  f32x2 acc2[P];
  float l = 0.f;
#pragma unroll
  for (int i = 0; i < P; ++i) acc2[i] = pk2(0.f, 0.f);

  // Every thread moves the 16-byte pieces it will use itself from the caches into its own slots of a shared-memory ring
  // with asynchronous copies, kStages - 1 steps ahead of their use: the loads of several steps are in flight while one
  // step is being summed, and no thread ever waits for another.  Pieces past the end of the key range are written as
  // zeros without touching memory (source size 0) and weigh nothing.
  extern __shared__ uint4 ring[];              // [kStages][kUnroll][2][kDecThreads]
  constexpr int kRows = kStep * kUnroll;       // key rows a CTA handles per step
  const int w_first = lo + warp * RPW;         // the same for the whole warp, and so are the trip counts
  const int j_first = w_first + g;
  const int n_steps = hi > w_first ? (hi - w_first + kRows - 1) / kRows : 0;
  const T* k_src = kc + j_first * p.kcs[2] + c * W;          // this thread's piece of the next step to be requested
  const T* v_src = vc + j_first * p.vcs[2] + c * W;
  const int64_t k_row = int64_t(kStep) * p.kcs[2], v_row = int64_t(kStep) * p.vcs[2];
  const uint32_t ring0 = uint32_t(__cvta_generic_to_shared(ring + tid));
  constexpr uint32_t kStageBytes = kUnroll * 2 * kDecThreads * 16, kPieceBytes = kDecThreads * 16;
  auto issue = [&](int step) {
    if (step < n_steps) {
      const uint32_t dst = ring0 + uint32_t(step % kStages) * kStageBytes;
      const bool whole = w_first + (step + 1) * kRows <= hi;                 // every row of the step is in range (warp-uniform)
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const bool in = whole || j_first + step * kRows + u * kStep < hi;
        const T* ks = in ? k_src + u * k_row : kc;
        const T* vs = in ? v_src + u * v_row : vc;
        const uint32_t bytes = in ? 16u : 0u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (2 * u) * kPieceBytes), "l"(ks), "r"(bytes) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (2 * u + 1) * kPieceBytes), "l"(vs), "r"(bytes) : "memory");
      }
      k_src += kUnroll * k_row;
      v_src += kUnroll * v_row;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");       // one group per step, empty or not: the waits count groups
  };
  // After the transpose reduction lane c of a row group holds the score of row `my_u` of the step's four rows.
  const bool up_a = (c & (LPR / 2)) != 0, up_b = (c & (LPR / 4)) != 0;
  const int my_u = 2 * int(up_a) + int(up_b);
  const int group0 = lane & ~(LPR - 1);
#pragma unroll
  for (int s0 = 0; s0 < kStages - 1; ++s0) issue(s0);
  for (int step = 0; step < n_steps; ++step) {
    issue(step + kStages - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 1) : "memory");     // this step's pieces have landed
    const uint4* slot = ring + size_t(step % kStages) * (kUnroll * 2 * kDecThreads) + tid;
    float d[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {        // this lane's share of the four dot products
      f32x2 k2[P];
      Pairs<T>::get(slot[(2 * u) * kDecThreads], k2);
      f32x2 t = pk2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < P; ++i) t = fma2(q2[i], k2[i], t);
      float t0, t1;
      upk2(t, t0, t1);
      d[u] = t0 + t1;
    }
    // four sums over LPR lanes at the price of little more than one: halve the rows while doubling the lanes summed
    const float a0 = (up_a ? d[2] : d[0]) + __shfl_xor_sync(0xffffffffu, up_a ? d[0] : d[2], LPR / 2);
    const float a1 = (up_a ? d[3] : d[1]) + __shfl_xor_sync(0xffffffffu, up_a ? d[1] : d[3], LPR / 2);
    float x = (up_b ? a1 : a0) + __shfl_xor_sync(0xffffffffu, up_b ? a0 : a1, LPR / 4);
#pragma unroll
    for (int o = LPR / 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    const int j = j_first + step * kRows + my_u * kStep;
    const float s = x - slope * float(n - j);
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fabsf(s) + 1.0f));
    const float sig = fmaf(s * r, 0.5f, 0.5f);
    const float sg2 = sig * sig;
    const float f = j < hi ? sg2 * sg2 : 0.f;
    l += f;                                    // (every row is counted by LPR/4 lanes; undone after the loop)
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const float fu = __shfl_sync(0xffffffffu, f, group0 + (u >> 1) * (LPR / 2) + (u & 1) * (LPR / 4));
      const f32x2 f2 = pk2(fu, fu);
      f32x2 v2[P];
      Pairs<T>::get(slot[(2 * u + 1) * kDecThreads], v2);
#pragma unroll
      for (int i = 0; i < P; ++i) acc2[i] = fma2(f2, v2[i], acc2[i]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  float acc[W];
#pragma unroll
  for (int i = 0; i < P; ++i) upk2(acc2[i], acc[2 * i], acc[2 * i + 1]);
#pragma unroll
  for (int o = LPR / 8; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);   // lanes that hold the other rows' weights
  l += __shfl_xor_sync(0xffffffffu, l, LPR / 4);
  l += __shfl_xor_sync(0xffffffffu, l, LPR / 2);
  l *= 4.0f / float(LPR);
  // rows of one warp -> one row
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
    for (int i = 0; i < W; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  if (g == 0) {
#pragma unroll
    for (int i = 0; i < W; ++i) red[warp][c * W + i] = acc[i];
    if (c == 0) red[warp][D] = l;
  }
  __syncthreads();
  for (int e = tid; e <= D; e += kDecThreads) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) t += red[w][e];
    tot[e] = t;
  }
  cluster.sync();                              // every CTA's totals are in its shared memory
  if (split == 0) {
    for (int e = tid; e < D; e += kDecThreads) {
      float a = 0.f, L = 0.f;
      for (int r = 0; r < n_split; ++r) {
        const float* remote = cluster.map_shared_rank(tot, r);
        a += remote[e];
        L += remote[D];
      }
      static_cast<T*>(p.out)[b * p.os[0] + h * p.os[1] + e] = Elem<T>::from_c(a / (L + p.eps));
    }
  }
  cluster.sync();                              // nobody leaves while the first CTA still reads its totals
}

template <typename T, int D>
int launch_decode(const DecodeParams& p, int n_split, cudaStream_t st) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(n_split), unsigned(p.B * p.H), 1);
  cfg.blockDim = dim3(kDecThreads, 1, 1);
  cfg.dynamicSmemBytes = kRingBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = unsigned(n_split);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  static bool configured = false;               // (per instantiation; racing threads set the same value)
  if (!configured) {
    cudaFuncSetAttribute(attn_decode_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    configured = true;
  }
  cudaLaunchKernelEx(&cfg, attn_decode_kernel<T, D>, p);
  return check_launch("attn_decode");
}

template <typename T>
int decode_t(const DecodeParams& p, int D, int n_split, cudaStream_t st) {
  switch (D) {
    case 32: return launch_decode<T, 32>(p, n_split, st);
    case 64: return launch_decode<T, 64>(p, n_split, st);
    case 128: return launch_decode<T, 128>(p, n_split, st);
    default: set_error("attn_decode: head size %d is not one of 32, 64, 128", D); return FAT_ERR_UNSUPPORTED;
  }
}

bool mult(const int64_t* s, int n, int w) {
  for (int i = 0; i < n; ++i) if (s[i] % w) return false;
  return true;
}

}  // namespace
}  // namespace fat

using namespace fat;

extern "C" int fat_attn_decode(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                               const int32_t* n_cached, const float* slopes, void* out, int B, int H, int capacity, int D,
                               const int64_t* q_strides, const int64_t* k_new_strides, const int64_t* v_new_strides,
                               const int64_t* out_strides, const int64_t* k_cache_strides, const int64_t* v_cache_strides,
                               double scale, double eps, int dtype, int* status, void* stream) {
  if (B < 0 || H <= 0 || capacity <= 0 || D <= 0 || int64_t(B) * H > 65535) {
    set_error("attn_decode: bad shape [B=%d, H=%d, capacity=%d, D=%d] (B*H must not exceed 65535)", B, H, capacity, D);
    return FAT_ERR_SHAPE;
  }
  if (B == 0) return FAT_OK;
  if (!q || !k_new || !v_new || !k_cache || !v_cache || !n_cached || !slopes || !out || !q_strides || !k_new_strides ||
      !v_new_strides || !out_strides || !k_cache_strides || !v_cache_strides) {
    set_error("attn_decode: null pointer");
    return FAT_ERR_NULL;
  }
  const int w = dtype == FAT_F32 ? 4 : 8;
  if (!aligned16(q) || !aligned16(k_new) || !aligned16(v_new) || !aligned16(k_cache) || !aligned16(v_cache) ||
      !mult(q_strides, 2, w) || !mult(k_new_strides, 2, w) || !mult(v_new_strides, 2, w) || !mult(k_cache_strides, 3, w) ||
      !mult(v_cache_strides, 3, w)) {
    set_error("attn_decode: q, the new rows and the caches must be 16-byte aligned with strides that are multiples of %d elements", w);
    return FAT_ERR_ALIGNMENT;
  }
  DecodeParams p{};
  p.q = q; p.k_new = k_new; p.v_new = v_new; p.k_cache = k_cache; p.v_cache = v_cache; p.n_cached = n_cached;
  p.slopes = slopes; p.out = out; p.B = B; p.H = H; p.capacity = capacity;
  for (int i = 0; i < 2; ++i) { p.qs[i] = q_strides[i]; p.kns[i] = k_new_strides[i]; p.vns[i] = v_new_strides[i]; p.os[i] = out_strides[i]; }
  for (int i = 0; i < 3; ++i) { p.kcs[i] = k_cache_strides[i]; p.vcs[i] = v_cache_strides[i]; }
  p.scale = float(scale); p.eps = float(eps); p.status = status;
  // enough CTAs to fill the GPU (FAT_DEC_FILL per SM), but no CTA with less than FAT_DEC_MIN_ROWS rows of a full cache
  int n_split = 1;
  while (n_split < 8 && int64_t(B) * H * n_split < FAT_DEC_FILL * int64_t(num_sms()) && capacity / (2 * n_split) >= FAT_DEC_MIN_ROWS) n_split *= 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FAT_F32: return decode_t<float>(p, D, n_split, st);
    case FAT_BF16: return decode_t<__nv_bfloat16>(p, D, n_split, st);
    case FAT_F16: return decode_t<__half>(p, D, n_split, st);
    default: set_error("attn_decode: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE;
  }
}
