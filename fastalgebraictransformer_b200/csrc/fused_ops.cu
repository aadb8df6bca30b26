// Bandwidth-bound kernels of the Algebraic-Transformer hot path for sm_100a:
// rational SwiGLU, mean-error normalisation and rational softmax, forward and backward.
//
// Design: every tensor is touched exactly once per kernel.  Rows are held in registers
// (16-byte packs, VPT packs per thread, G threads per row, 256/G rows per block) so the
// row statistics and the output come from a single read; reductions are warp shuffles
// plus one shared-memory hop when a row spans several warps.  Loads and stores carry
// streaming hints (read-once / write-once data should not displace L2 contents).
// Shapes or alignments that do not fit the register-resident scheme go through "slow"
// kernels (one block per row, two passes, scalar accesses) that accept anything.
#include <initializer_list>
#include <mutex>

#include "common.cuh"

namespace fat {
namespace {

// Launch-shape constants (blocks per SM that the grids are sized for, 16-byte loads in flight per thread
// and tensor); the values were picked by sweeping them on a B200.
#ifndef FAT_NORM_FWD_BPS
#define FAT_NORM_FWD_BPS 8
#define FAT_NORM_FWD_PPT 2
#define FAT_NORM_BWD_BPS 2
#define FAT_NORM_BWD_PPT 2
#define FAT_SOFTMAX_BPS 6
#define FAT_SOFTMAX_PPT 4
#define FAT_SWIGLU_BPS 24
#endif

constexpr int kThreads = 256;
constexpr int kMaxVPT = 8;
// rows of the d_weight partial-sum scratch: one per block of the norm backward, whose grid never exceeds this
inline int norm_bwd_max_blocks() { return FAT_NORM_BWD_BPS * num_sms(); }

// Scratch of fat_norm_bwd_static: a fixed array inside the library image.  Every GPU that loads
// the library holds these 16 MiB until the process exits; all calls on a device share them.
constexpr size_t kStaticScratchBytes = size_t(16) << 20;
constexpr int kMaxDevices = 64;

// ------------------------------------------------------------------ group reduction
// Sums NV values over the G threads (G = 32..256, power of two) that share a row.
// `buf` is shared memory of 2*(NT/32)*NV values; `phase` alternates the half in use so that one
// __syncthreads per call suffices.  Every thread of the block must call it.
template <typename C, int NV, int NT = 256>
__device__ __forceinline__ void group_sum(C (&v)[NV], int G, C* buf, int& phase) {
#pragma unroll
  for (int n = 0; n < NV; ++n) v[n] = warp_sum(v[n]);
  if (G > 32) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    C* b = buf + phase * (NT / 32) * NV;
    if (lane == 0) {
#pragma unroll
      for (int n = 0; n < NV; ++n) b[warp * NV + n] = v[n];
    }
    __syncthreads();
    const int wpg = G >> 5, w0 = (warp / wpg) * wpg;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      C s = C(0);
      for (int w = 0; w < wpg; ++w) s += b[(w0 + w) * NV + n];
      v[n] = s;
    }
    phase ^= 1;
  }
}

// =====================================================================================
// SwiGLU
// =====================================================================================
template <typename T, int W>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ value, T* __restrict__ out,
                  int64_t n_rows, int64_t packs_per_row, int64_t gs, int64_t vs, int64_t os) {
  using C = typename Elem<T>::C;
  const int64_t step = int64_t(gridDim.x) * kThreads;
  for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
    const T* g = gate + row * gs; const T* v = value + row * vs; T* o = out + row * os;
#pragma unroll 4
    for (int64_t pk = int64_t(blockIdx.x) * kThreads + threadIdx.x; pk < packs_per_row; pk += step) {
      C a[W], b[W], r[W];
      load_pack<T, W>(g + pk * W, a);
      load_pack<T, W>(v + pk * W, b);
#pragma unroll
      for (int i = 0; i < W; ++i) r[i] = a[i] * rsigmoid(a[i], rcp1p_abs(a[i])) * b[i];
      store_pack<T, W>(o + pk * W, r);
    }
  }
}

template <typename T, int W>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_kernel(const T* __restrict__ d_out, const T* __restrict__ gate, const T* __restrict__ value,
                  T* __restrict__ d_gate, T* __restrict__ d_value,
                  int64_t n_rows, int64_t packs_per_row,
                  int64_t dos, int64_t gs, int64_t vs, int64_t dgs, int64_t dvs) {
  using C = typename Elem<T>::C;
  const int64_t step = int64_t(gridDim.x) * kThreads;
  for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
    const T* go = d_out + row * dos; const T* g = gate + row * gs; const T* v = value + row * vs;
    T* dg = d_gate + row * dgs; T* dv = d_value + row * dvs;
#pragma unroll 2
    for (int64_t pk = int64_t(blockIdx.x) * kThreads + threadIdx.x; pk < packs_per_row; pk += step) {
      C o[W], a[W], b[W], ra[W], rb[W];
      load_pack<T, W>(go + pk * W, o);
      load_pack<T, W>(g + pk * W, a);
      load_pack<T, W>(v + pk * W, b);
#pragma unroll
      for (int i = 0; i < W; ++i) {
        const C r = rcp1p_abs(a[i]);
        const C s = rsigmoid(a[i], r);
        rb[i] = o[i] * a[i] * s;                              // d_value = d_out * gate * sigma
        ra[i] = o[i] * b[i] * (s + a[i] * C(0.5) * r * r);    // d_gate  = d_out * value * (sigma + gate sigma')
      }
      store_pack<T, W>(dg + pk * W, ra);
      store_pack<T, W>(dv + pk * W, rb);
    }
  }
}

// =====================================================================================
// Register-resident row kernels (fast path)
// =====================================================================================
// The packs of one row as they come from memory.  Rows are fetched one iteration ahead: the loads of
// the next row are issued before the current row's reduction (which ends in a block-wide barrier), so
// memory stays busy across the barrier.
template <typename T, int VPT>
struct RawRow {
  static constexpr int W = 16 / sizeof(T);
  uint4 v[VPT];
  __device__ __forceinline__ void fetch(const T* row, int t, int G, int npk, bool ok) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int pk = t + i * G;
      v[i] = (ok && pk < npk) ? __ldcs(reinterpret_cast<const uint4*>(row + int64_t(pk) * W)) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
};

template <typename T, int W, int VPT>
struct RowRegs {
  using C = typename Elem<T>::C;
  C v[VPT][W];
  __device__ __forceinline__ void from_raw(const RawRow<T, VPT>& raw) {     // all-zero bits are 0.0 in every element type
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const T* e = reinterpret_cast<const T*>(&raw.v[i]);
#pragma unroll
      for (int j = 0; j < W; ++j) v[i][j] = Elem<T>::to_c(e[j]);
    }
  }
  __device__ __forceinline__ void load(const T* row, int t, int G, int npk, bool ok) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int pk = t + i * G;
      if (ok && pk < npk) load_pack<T, W>(row + int64_t(pk) * W, v[i]);
      else {
#pragma unroll
        for (int j = 0; j < W; ++j) v[i][j] = C(0);
      }
    }
  }
};

// ADD: the normalised row is h = x + res, rounded to the tensor dtype and also written to h_out (the residual stream
// of a pre-norm block: one pass instead of an addition pass followed by a normalisation pass).
template <typename T, int W, int VPT, bool ADD = false>
__global__ void __launch_bounds__(kThreads)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ weight, T* __restrict__ y,
                float* __restrict__ mean, int64_t n_rows, int n_cols, int64_t xs, int64_t ys,
                double eps_d, int G, const T* __restrict__ res = nullptr, T* __restrict__ h_out = nullptr,
                int64_t rs = 0, int64_t hs = 0) {
  using C = typename Elem<T>::C;
  __shared__ C red[2 * (kThreads / 32)];
  int phase = 0;
  const int npk = n_cols / W, rpc = kThreads / G, g = threadIdx.x / G, t = threadIdx.x % G;
  const C eps = C(eps_d);
  C w[VPT][W];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int pk = t + i * G;
    if (pk < npk) load_pack_cached<T, W>(weight + int64_t(pk) * W, w[i]);
  }
  const int64_t row_step = int64_t(gridDim.x) * rpc, first_row = int64_t(blockIdx.x) * rpc + g;
  RawRow<T, VPT> next_x, next_r;
  next_x.fetch(x + first_row * xs, t, G, npk, first_row < n_rows);
  if (ADD) next_r.fetch(res + first_row * rs, t, G, npk, first_row < n_rows);
  for (int64_t row0 = int64_t(blockIdx.x) * rpc; row0 < n_rows; row0 += int64_t(gridDim.x) * rpc) {
    const int64_t row = row0 + g;
    const bool ok = row < n_rows;
    RowRegs<T, W, VPT> xr;
    xr.from_raw(next_x);
    next_x.fetch(x + (row + row_step) * xs, t, G, npk, row + row_step < n_rows);
    if (ADD) {
      RowRegs<T, W, VPT> rr;
      rr.from_raw(next_r);
      next_r.fetch(res + (row + row_step) * rs, t, G, npk, row + row_step < n_rows);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int j = 0; j < W; ++j)      // the sum as it is stored: the normalisation sees exactly what the next reader of h_out sees
          xr.v[i][j] = Elem<T>::to_c(Elem<T>::from_c(xr.v[i][j] + rr.v[i][j]));
        const int pk = t + i * G;
        if (ok && pk < npk) store_pack<T, W>(h_out + row * hs + int64_t(pk) * W, xr.v[i]);
      }
    }
    C s[1] = {C(0)};
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < W; ++j) s[0] += fabs(xr.v[i][j]);
    group_sum<C, 1>(s, G, red, phase);
    const C m = s[0] / C(n_cols);
    const C inv = C(1) / (m + eps);
    if (ok) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int pk = t + i * G;
        if (pk < npk) {
          C o[W];
#pragma unroll
          for (int j = 0; j < W; ++j) o[j] = xr.v[i][j] * inv * w[i][j];
          store_pack<T, W>(y + row * ys + int64_t(pk) * W, o);
        }
      }
      if (t == 0) mean[row] = float(m);
    }
  }
}

// d_x for every row, plus this block's partial column sums of d_out * x / mu into
// partial[blockIdx.x][0..n_cols) (compute type).  To leave registers for rows in flight the weight stays
// packed (converted where used) and the running column sums live in thread-private shared-memory slots.
// dyn smem: NT * VPT * W values.
// ADD: d_x additionally receives d_add (the gradient that reached the normalised tensor along the residual path).
template <typename T, int W, int VPT, int NT, bool ADD = false>
__global__ void __launch_bounds__(NT)
norm_bwd_kernel(const T* __restrict__ d_out, const T* __restrict__ x, const T* __restrict__ weight,
                const float* __restrict__ mean, T* __restrict__ d_x,
                typename Elem<T>::C* __restrict__ partial,
                int64_t n_rows, int n_cols, int64_t dos, int64_t xs, int64_t dxs,
                double eps_d, int G, const T* __restrict__ d_add = nullptr, int64_t das = 0) {
  using C = typename Elem<T>::C;
  __shared__ C red[2 * (NT / 32)];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  C* acc_sm = reinterpret_cast<C*>(dyn_smem);            // slot (i, j) of thread tid: acc_sm[(i * W + j) * NT + tid]
  int phase = 0;
  const int npk = n_cols / W, rpc = NT / G, g = threadIdx.x / G, t = threadIdx.x % G;
  const C eps = C(eps_d);
  RawRow<T, VPT> wraw;
  wraw.fetch(weight, t, G, npk, true);
#pragma unroll
  for (int i = 0; i < VPT * W; ++i) acc_sm[i * NT + threadIdx.x] = C(0);
  const int64_t row_step = int64_t(gridDim.x) * rpc, first_row = int64_t(blockIdx.x) * rpc + g;
  RawRow<T, VPT> next_x;
  next_x.fetch(x + first_row * xs, t, G, npk, first_row < n_rows);
  RawRow<T, VPT> next_g;
  next_g.fetch(d_out + first_row * dos, t, G, npk, first_row < n_rows);
  float next_mean = first_row < n_rows ? __ldg(mean + first_row) : 0.f;       // fetched a row ahead like the packs
  for (int64_t row0 = int64_t(blockIdx.x) * rpc; row0 < n_rows; row0 += int64_t(gridDim.x) * rpc) {
    const int64_t row = row0 + g;
    const bool ok = row < n_rows;
    RowRegs<T, W, VPT> xr;
    xr.from_raw(next_x);
    next_x.fetch(x + (row + row_step) * xs, t, G, npk, row + row_step < n_rows);
    RowRegs<T, W, VPT> gr;
    gr.from_raw(next_g);
    next_g.fetch(d_out + (row + row_step) * dos, t, G, npk, row + row_step < n_rows);
    const C inv = ok ? C(1) / (C(next_mean) + eps) : C(0);
    next_mean = row + row_step < n_rows ? __ldg(mean + row + row_step) : 0.f;
    C s[1] = {C(0)};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const T* we = reinterpret_cast<const T*>(&wraw.v[i]);
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const C gxn = gr.v[i][j] * (xr.v[i][j] * inv);      // d_out * x / mu  (0 beyond the row: zero packs)
        acc_sm[(i * W + j) * NT + threadIdx.x] += gxn;
        s[0] += gxn * Elem<T>::to_c(we[j]);
      }
    }
    group_sum<C, 1, NT>(s, G, red, phase);
    const C corr = s[0] / C(n_cols) * inv;
    if (ok) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int pk = t + i * G;
        if (pk < npk) {
          const T* we = reinterpret_cast<const T*>(&wraw.v[i]);
          C o[W];
#pragma unroll
          for (int j = 0; j < W; ++j)
            o[j] = gr.v[i][j] * Elem<T>::to_c(we[j]) * inv - sgn(xr.v[i][j]) * corr;
          if (ADD) {
            C a[W];
            load_pack<T, W>(d_add + row * das + int64_t(pk) * W, a);
#pragma unroll
            for (int j = 0; j < W; ++j) o[j] = Elem<T>::to_c(Elem<T>::from_c(o[j])) + a[j];   // rounded like the separate norm backward, then added
          }
          store_pack<T, W>(d_x + row * dxs + int64_t(pk) * W, o);
        }
      }
    }
  }
  // fold the row groups of this block and publish the block's partial sums
  C* prow = partial + int64_t(blockIdx.x) * n_cols;
  __syncthreads();
  for (int c = threadIdx.x; c < n_cols; c += NT) {
    const int pk = c / W, j = c % W, i = pk / G, tt = pk % G;
    C sum = C(0);
    for (int r = 0; r < rpc; ++r) sum += acc_sm[(i * W + j) * NT + r * G + tt];
    prow[c] = sum;
  }
}

// ---------------------------------------------------------------- 16-bit rows, packed float32 arithmetic
// The same backward for bfloat16 / float16 rows of up to two 16-byte packs per thread, written for instruction count:
// the generic kernel above spends ~30 instructions per element (scalar conversions, a shared-memory read-modify-write
// per element for the column sums, the weight converted twice per row) and is bound by instruction issue, not by
// memory.  Here two neighbouring elements travel as one float32 pair (fma.rn.f32x2 and friends), the weight is
// unpacked once per block, and the running column sums stay in registers until the block is done.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// one 32-bit word holding two 16-bit elements -> the pair as float32 (element 0 first)
template <typename T> __device__ __forceinline__ void unpack16(uint32_t w, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16); hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack16<__half>(uint32_t w, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w)); lo = f.x; hi = f.y;
}
template <typename T> __device__ __forceinline__ uint32_t pack16(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack16<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v);
}
// -sign(x) * c with sign(0) = 0 (c given as the bits of -c)
__device__ __forceinline__ float neg_signed(float x, uint32_t neg_c_bits) {
  const float v = __uint_as_float((__float_as_uint(x) & 0x80000000u) ^ neg_c_bits);
  return x == 0.f ? 0.f : v;
}

#ifndef FAT_NORM_BWD16_MINB
#define FAT_NORM_BWD16_MINB 2
#endif
template <typename T, int VPT, int NT, bool ADD = false>
__global__ void __launch_bounds__(NT, NT == 256 ? FAT_NORM_BWD16_MINB : 1)
norm_bwd16_kernel(const T* __restrict__ d_out, const T* __restrict__ x, const T* __restrict__ weight,
                  const float* __restrict__ mean, T* __restrict__ d_x, float* __restrict__ partial,
                  int64_t n_rows, int n_cols, int64_t dos, int64_t xs, int64_t dxs,
                  double eps_d, int G, const T* __restrict__ d_add = nullptr, int64_t das = 0) {
  constexpr int W = 8;
  __shared__ float red[2 * (NT / 32)];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  float* acc_sm = reinterpret_cast<float*>(dyn_smem);     // used once, at the end: slot (i, j) of thread tid at [(i * W + j) * NT + tid]
  int phase = 0;
  const int npk = n_cols / W, rpc = NT / G, g = threadIdx.x / G, t = threadIdx.x % G;
  const float eps = float(eps_d);
  f32x2 w2[VPT][4], acc[VPT][4];
  {
    RawRow<T, VPT> wraw;
    wraw.fetch(weight, t, G, npk, true);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wraw.v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) { float a, b; unpack16<T>(ww[k], a, b); w2[i][k] = pk2(a, b); acc[i][k] = pk2(0.f, 0.f); }
    }
  }
  const int64_t row_step = int64_t(gridDim.x) * rpc, first_row = int64_t(blockIdx.x) * rpc + g;
  RawRow<T, VPT> next_x, next_g, next_a;
  next_x.fetch(x + first_row * xs, t, G, npk, first_row < n_rows);
  next_g.fetch(d_out + first_row * dos, t, G, npk, first_row < n_rows);
  if (ADD) next_a.fetch(d_add + first_row * das, t, G, npk, first_row < n_rows);
  float next_mean = first_row < n_rows ? __ldg(mean + first_row) : 0.f;       // fetched a row ahead like the packs
  for (int64_t row0 = int64_t(blockIdx.x) * rpc; row0 < n_rows; row0 += row_step) {
    const int64_t row = row0 + g;
    const bool ok = row < n_rows;
    const RawRow<T, VPT> xr = next_x, gr = next_g;
    RawRow<T, VPT> ar;
    if (ADD) ar = next_a;
    const bool more = row + row_step < n_rows;
    next_x.fetch(x + (row + row_step) * xs, t, G, npk, more);
    next_g.fetch(d_out + (row + row_step) * dos, t, G, npk, more);
    if (ADD) next_a.fetch(d_add + (row + row_step) * das, t, G, npk, more);
    const float inv = ok ? 1.0f / (next_mean + eps) : 0.f;
    next_mean = more ? __ldg(mean + row + row_step) : 0.f;
    const f32x2 inv2 = pk2(inv, inv);
    f32x2 s2 = pk2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xr.v[i]);
      const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gr.v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float x0, x1, g0, g1;
        unpack16<T>(xw[k], x0, x1);
        unpack16<T>(gw[k], g0, g1);
        const f32x2 gxn = mul2(pk2(g0, g1), mul2(pk2(x0, x1), inv2));     // d_out * x / mu  (0 beyond the row: zero packs)
        acc[i][k] = add2(acc[i][k], gxn);
        s2 = fma2(gxn, w2[i][k], s2);
      }
    }
    float s[1];
    {
      float a, b;
      upk2(s2, a, b);
      s[0] = a + b;
    }
    group_sum<float, 1, NT>(s, G, red, phase);
    const float corr = s[0] / float(n_cols) * inv;
    const uint32_t neg_corr = __float_as_uint(-corr);
    if (ok) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int pk = t + i * G;
        if (pk < npk) {
          const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xr.v[i]);
          const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gr.v[i]);
          const uint32_t* aw = reinterpret_cast<const uint32_t*>(&ar.v[i]);
          uint4 out_raw;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&out_raw);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float x0, x1, g0, g1, o0, o1;
            unpack16<T>(xw[k], x0, x1);
            unpack16<T>(gw[k], g0, g1);
            // d_out * w / mu - sign(x) * corr
            upk2(fma2(mul2(pk2(g0, g1), w2[i][k]), inv2, pk2(neg_signed(x0, neg_corr), neg_signed(x1, neg_corr))), o0, o1);
            uint32_t packed = pack16<T>(o0, o1);
            if (ADD) {                                       // rounded like the separate norm backward, then added
              float r0, r1, a0, a1;
              unpack16<T>(packed, r0, r1);
              unpack16<T>(aw[k], a0, a1);
              packed = pack16<T>(r0 + a0, r1 + a1);
            }
            ow[k] = packed;
          }
          __stcs(reinterpret_cast<uint4*>(d_x + row * dxs + int64_t(pk) * W), out_raw);
        }
      }
    }
  }
  // fold the row groups of this block and publish the block's partial sums
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a, b;
      upk2(acc[i][k], a, b);
      acc_sm[(i * W + 2 * k) * NT + threadIdx.x] = a;
      acc_sm[(i * W + 2 * k + 1) * NT + threadIdx.x] = b;
    }
  }
  float* prow = partial + int64_t(blockIdx.x) * n_cols;
  __syncthreads();
  for (int c = threadIdx.x; c < n_cols; c += NT) {
    const int pk = c / W, j = c % W, i = pk / G, tt = pk % G;
    float sum = 0.f;
    for (int r = 0; r < rpc; ++r) sum += acc_sm[(i * W + j) * NT + r * G + tt];
    prow[c] = sum;
  }
}

// d_weight[c] = sum over the n_part partial rows.  Block = 32 columns x kReduceSlices slices of the partial rows,
// so that a thread has only a handful of (independent) loads to wait for.
constexpr int kReduceSlices = 32;
template <typename T>
__global__ void __launch_bounds__(32 * kReduceSlices)
norm_bwd_reduce_kernel(const typename Elem<T>::C* __restrict__ partial, T* __restrict__ d_weight,
                       int n_part, int n_cols) {
  using C = typename Elem<T>::C;
  __shared__ C sm[kReduceSlices][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  C s = C(0);
  if (c < n_cols) {
#pragma unroll 8
    for (int r = slice; r < n_part; r += kReduceSlices) s += partial[int64_t(r) * n_cols + c];
  }
  sm[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && c < n_cols) {
#pragma unroll
    for (int r = 1; r < kReduceSlices; ++r) s += sm[r][lane];
    d_weight[c] = Elem<T>::from_c(s);
  }
}

template <typename T, int W, int VPT>
__global__ void __launch_bounds__(kThreads)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ p, int64_t n_rows, int n_cols,
                   int64_t xs, int64_t ps, double eps_d, int G) {
  using C = typename Elem<T>::C;
  __shared__ C red[2 * (kThreads / 32)];
  int phase = 0;
  const int npk = n_cols / W, rpc = kThreads / G, g = threadIdx.x / G, t = threadIdx.x % G;
  const C eps = C(eps_d);
  const int64_t row_step = int64_t(gridDim.x) * rpc, first_row = int64_t(blockIdx.x) * rpc + g;
  RawRow<T, VPT> next_x;
  next_x.fetch(x + first_row * xs, t, G, npk, first_row < n_rows);
  for (int64_t row0 = int64_t(blockIdx.x) * rpc; row0 < n_rows; row0 += int64_t(gridDim.x) * rpc) {
    const int64_t row = row0 + g;
    const bool ok = row < n_rows;
    RowRegs<T, W, VPT> xr;
    xr.from_raw(next_x);
    next_x.fetch(x + (row + row_step) * xs, t, G, npk, row + row_step < n_rows);
    C s[1] = {C(0)};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const bool live = t + i * G < npk;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const C v = xr.v[i][j];
        C f = rsigmoid(v, rcp1p_abs(v));
        f *= f; f *= f;
        f = live ? f : C(0);
        xr.v[i][j] = f;                 // the row now holds sigma^4
        s[0] += f;
      }
    }
    group_sum<C, 1>(s, G, red, phase);
    const C inv = C(1) / (s[0] + eps);
    if (ok) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int pk = t + i * G;
        if (pk < npk) {
          C o[W];
#pragma unroll
          for (int j = 0; j < W; ++j) o[j] = xr.v[i][j] * inv;
          store_pack<T, W>(p + row * ps + int64_t(pk) * W, o);
        }
      }
    }
  }
}

template <typename T, int W, int VPT>
__global__ void __launch_bounds__(kThreads)
softmax_bwd_kernel(const T* __restrict__ d_out, const T* __restrict__ x, T* __restrict__ d_x,
                   int64_t n_rows, int n_cols, int64_t dos, int64_t xs, int64_t dxs,
                   double eps_d, int G) {
  using C = typename Elem<T>::C;
  __shared__ C red[2 * (kThreads / 32) * 2];
  int phase = 0;
  const int npk = n_cols / W, rpc = kThreads / G, g = threadIdx.x / G, t = threadIdx.x % G;
  const C eps = C(eps_d);
  const int64_t row_step = int64_t(gridDim.x) * rpc, first_row = int64_t(blockIdx.x) * rpc + g;
  RawRow<T, VPT> next_x;
  next_x.fetch(x + first_row * xs, t, G, npk, first_row < n_rows);
  RawRow<T, VPT> next_g;
  next_g.fetch(d_out + first_row * dos, t, G, npk, first_row < n_rows);
  for (int64_t row0 = int64_t(blockIdx.x) * rpc; row0 < n_rows; row0 += int64_t(gridDim.x) * rpc) {
    const int64_t row = row0 + g;
    const bool ok = row < n_rows;
    RowRegs<T, W, VPT> xr;
    xr.from_raw(next_x);
    next_x.fetch(x + (row + row_step) * xs, t, G, npk, row + row_step < n_rows);
    RowRegs<T, W, VPT> gr;
    gr.from_raw(next_g);
    next_g.fetch(d_out + (row + row_step) * dos, t, G, npk, row + row_step < n_rows);
    // after this loop xr holds k = 2 sigma^3 r^2 (the un-normalised derivative factor)
    C s[2] = {C(0), C(0)};                 // Z = sum sigma^4 ; sum d_out * sigma^4
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const bool live = t + i * G < npk;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const C v = xr.v[i][j];
        const C r = rcp1p_abs(v);
        const C sg = rsigmoid(v, r);
        const C s2 = sg * sg;
        const C f = live ? s2 * s2 : C(0);
        s[0] += f;
        s[1] += gr.v[i][j] * f;
        xr.v[i][j] = C(2) * s2 * sg * r * r;
      }
    }
    group_sum<C, 2>(s, G, red, phase);
    const C inv = C(1) / (s[0] + eps);
    const C dot = s[1] * inv;
    if (ok) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int pk = t + i * G;
        if (pk < npk) {
          C o[W];
#pragma unroll
          for (int j = 0; j < W; ++j) o[j] = xr.v[i][j] * inv * (gr.v[i][j] - dot);
          store_pack<T, W>(d_x + row * dxs + int64_t(pk) * W, o);
        }
      }
    }
  }
}

// =====================================================================================
// Slow path: one block per row, two passes, scalar accesses, any n_cols / alignment
// =====================================================================================
enum RowOp { kNormFwd, kNormBwd, kSoftmaxFwd, kSoftmaxBwd };

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
row_slow_kernel(const T* __restrict__ a,      // x
                const T* __restrict__ b,      // d_out (bwd ops) or unused
                const T* __restrict__ weight, // norm ops
                float* __restrict__ mean_out, const float* __restrict__ mean_in,
                T* __restrict__ out, typename Elem<T>::C* __restrict__ partial,
                int64_t n_rows, int64_t n_cols, int64_t as, int64_t bs, int64_t os, double eps_d) {
  using C = typename Elem<T>::C;
  __shared__ C red[2 * (kThreads / 32) * 2];
  int phase = 0;
  const C eps = C(eps_d);
  if (OP == kNormBwd)
    for (int64_t c = threadIdx.x; c < n_cols; c += kThreads) partial[int64_t(blockIdx.x) * n_cols + c] = C(0);
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const T* x = a + row * as;
    const T* go = b ? b + row * bs : nullptr;
    T* o = out + row * os;
    C s[2] = {C(0), C(0)};
    C inv = C(0);
    if (OP == kNormBwd) inv = C(1) / (C(mean_in[row]) + eps);
    for (int64_t c = threadIdx.x; c < n_cols; c += kThreads) {
      const C v = Elem<T>::to_c(x[c]);
      if (OP == kNormFwd) s[0] += fabs(v);
      if (OP == kNormBwd) s[0] += Elem<T>::to_c(go[c]) * (v * inv) * Elem<T>::to_c(weight[c]);
      if (OP == kSoftmaxFwd || OP == kSoftmaxBwd) {
        C f = rsigmoid(v, rcp1p_abs(v)); f *= f; f *= f;
        s[0] += f;
        if (OP == kSoftmaxBwd) s[1] += Elem<T>::to_c(go[c]) * f;
      }
    }
    group_sum<C, 2>(s, kThreads, red, phase);
    if (OP == kNormFwd) {
      const C m = s[0] / C(n_cols);
      inv = C(1) / (m + eps);
      if (threadIdx.x == 0) mean_out[row] = float(m);
    }
    if (OP == kSoftmaxFwd || OP == kSoftmaxBwd) inv = C(1) / (s[0] + eps);
    for (int64_t c = threadIdx.x; c < n_cols; c += kThreads) {
      const C v = Elem<T>::to_c(x[c]);
      C r;
      if (OP == kNormFwd) r = v * inv * Elem<T>::to_c(weight[c]);
      if (OP == kNormBwd) {
        const C g = Elem<T>::to_c(go[c]);
        r = g * Elem<T>::to_c(weight[c]) * inv - sgn(v) * (s[0] / C(n_cols) * inv);
        partial[int64_t(blockIdx.x) * n_cols + c] += g * (v * inv);
      }
      if (OP == kSoftmaxFwd) { C f = rsigmoid(v, rcp1p_abs(v)); f *= f; f *= f; r = f * inv; }
      if (OP == kSoftmaxBwd) {
        const C rr = rcp1p_abs(v); const C sg = rsigmoid(v, rr);
        r = C(2) * sg * sg * sg * rr * rr * inv * (Elem<T>::to_c(go[c]) - s[1] * inv);
      }
      o[c] = Elem<T>::from_c(r);
    }
  }
}

// =====================================================================================
// Host-side dispatch
// =====================================================================================
struct RowPlan { bool fast; int G; int vpt; int grid; };

// Grid of a grid-stride kernel over `items` equal work items with at most `max_blocks` blocks: every block gets the
// same number of items (give or take one), so that no block is still working while the others have run out.  With
// the plain min(items, max_blocks), 2048 items on 888 blocks would leave 272 blocks with a third item while 616 idle.
inline int balanced_grid(int64_t items, int64_t max_blocks) {
  if (items <= max_blocks) return int(items);
  const int64_t per_block = (items + max_blocks - 1) / max_blocks;
  return int((items + per_block - 1) / per_block);
}

// Fast path: all pointers 16-byte aligned, n_cols and the row strides multiples of the pack
// width, and the row fits in registers (<= 256 * 8 packs).
template <typename T>
RowPlan plan_rows(int64_t n_rows, int64_t n_cols, std::initializer_list<const void*> ptrs,
                  std::initializer_list<int64_t> strides, int blocks_per_sm, int packs_per_thread = 2,
                  int threads = kThreads) {
  constexpr int W = 16 / sizeof(T);
  RowPlan p{true, 32, 1, 1};
  for (const void* q : ptrs) if (q && !aligned16(q)) p.fast = false;
  for (int64_t s : strides) if (s % W) p.fast = false;
  if (n_cols % W || n_cols / W > int64_t(threads) * kMaxVPT) p.fast = false;
  if (p.fast) {
    const int npk = int(n_cols / W);
    int G = 32;
    while (G < threads && (npk + G - 1) / G > packs_per_thread) G <<= 1;   // aim for this many 16-byte loads in flight per thread and tensor
    p.G = G;
    const int need = (npk + G - 1) / G;
    p.vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    const int rpc = threads / G;
    p.grid = balanced_grid((n_rows + rpc - 1) / rpc, int64_t(blocks_per_sm) * num_sms());
  } else {
    p.grid = balanced_grid(n_rows, int64_t(blocks_per_sm) * num_sms());
  }
  if (p.grid < 1) p.grid = 1;
  return p;
}

#define FAT_VPT_SWITCH(vpt, ...)                                  \
  switch (vpt) {                                                  \
    case 1: { constexpr int VPT = 1; __VA_ARGS__; } break;        \
    case 2: { constexpr int VPT = 2; __VA_ARGS__; } break;        \
    case 4: { constexpr int VPT = 4; __VA_ARGS__; } break;        \
    default: { constexpr int VPT = 8; __VA_ARGS__; } break;       \
  }

template <typename T>
int swiglu_fwd_t(const void* gate, const void* value, void* out, int64_t n_rows, int64_t n_cols,
                 int64_t gs, int64_t vs, int64_t os, cudaStream_t st) {
  constexpr int W = 16 / sizeof(T);
  if (gs == n_cols && vs == n_cols && os == n_cols) { n_cols *= n_rows; n_rows = 1; gs = vs = os = n_cols; }
  const bool vec = aligned16(gate) && aligned16(value) && aligned16(out) && n_cols % W == 0 &&
                   gs % W == 0 && vs % W == 0 && os % W == 0;
  const int64_t ppr = vec ? n_cols / W : n_cols;
  int64_t gx = (ppr + kThreads - 1) / kThreads;
  const int64_t cap = int64_t(FAT_SWIGLU_BPS) * num_sms();
  if (gx > cap) gx = cap;
  int64_t gy = n_rows < (cap + gx - 1) / gx ? n_rows : (cap + gx - 1) / gx;
  dim3 grid((unsigned)gx, (unsigned)gy);
  if (vec) swiglu_fwd_kernel<T, W><<<grid, kThreads, 0, st>>>((const T*)gate, (const T*)value, (T*)out, n_rows, ppr, gs, vs, os);
  else     swiglu_fwd_kernel<T, 1><<<grid, kThreads, 0, st>>>((const T*)gate, (const T*)value, (T*)out, n_rows, ppr, gs, vs, os);
  return check_launch("swiglu_fwd");
}

template <typename T>
int swiglu_bwd_t(const void* d_out, const void* gate, const void* value, void* d_gate, void* d_value,
                 int64_t n_rows, int64_t n_cols, int64_t dos, int64_t gs, int64_t vs, int64_t dgs, int64_t dvs,
                 cudaStream_t st) {
  constexpr int W = 16 / sizeof(T);
  if (dos == n_cols && gs == n_cols && vs == n_cols && dgs == n_cols && dvs == n_cols) {
    n_cols *= n_rows; n_rows = 1; dos = gs = vs = dgs = dvs = n_cols;
  }
  const bool vec = aligned16(d_out) && aligned16(gate) && aligned16(value) && aligned16(d_gate) && aligned16(d_value) &&
                   n_cols % W == 0 && dos % W == 0 && gs % W == 0 && vs % W == 0 && dgs % W == 0 && dvs % W == 0;
  const int64_t ppr = vec ? n_cols / W : n_cols;
  int64_t gx = (ppr + kThreads - 1) / kThreads;
  const int64_t cap = int64_t(FAT_SWIGLU_BPS) * num_sms();
  if (gx > cap) gx = cap;
  int64_t gy = n_rows < (cap + gx - 1) / gx ? n_rows : (cap + gx - 1) / gx;
  dim3 grid((unsigned)gx, (unsigned)gy);
  if (vec) swiglu_bwd_kernel<T, W><<<grid, kThreads, 0, st>>>((const T*)d_out, (const T*)gate, (const T*)value, (T*)d_gate, (T*)d_value, n_rows, ppr, dos, gs, vs, dgs, dvs);
  else     swiglu_bwd_kernel<T, 1><<<grid, kThreads, 0, st>>>((const T*)d_out, (const T*)gate, (const T*)value, (T*)d_gate, (T*)d_value, n_rows, ppr, dos, gs, vs, dgs, dvs);
  return check_launch("swiglu_bwd");
}

// out[r][c] = a[r][c] + b[r][c] (rounded once, like a tensor addition): the shapes the register kernels do not take
template <typename T>
__global__ void __launch_bounds__(kThreads)
add_rows_kernel(const T* a, const T* b, T* out, int64_t n_rows, int64_t n_cols,        // out may be a
                int64_t as, int64_t bs, int64_t os) {
  using C = typename Elem<T>::C;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x)
    for (int64_t c = threadIdx.x; c < n_cols; c += kThreads)
      out[row * os + c] = Elem<T>::from_c(Elem<T>::to_c(a[row * as + c]) + Elem<T>::to_c(b[row * bs + c]));
}

template <typename T>
int add_rows_t(const void* a, const void* b, void* out, int64_t n_rows, int64_t n_cols, int64_t as, int64_t bs, int64_t os,
               cudaStream_t st) {
  const int64_t cap = 32 * int64_t(num_sms());
  add_rows_kernel<T><<<unsigned(n_rows < cap ? n_rows : cap), kThreads, 0, st>>>((const T*)a, (const T*)b, (T*)out, n_rows,
                                                                                n_cols, as, bs, os);
  return check_launch("add_rows");
}

// res != nullptr: y = norm(x + res), h_out = x + res
template <typename T>
int norm_fwd_t(const void* x, const void* w, void* y, float* mean, int64_t n_rows, int64_t n_cols,
               int64_t xs, int64_t ys, double eps, cudaStream_t st,
               const void* res = nullptr, void* h_out = nullptr, int64_t rs = 0, int64_t hs = 0) {
  constexpr int W = 16 / sizeof(T);
  if (res) {
    RowPlan p = plan_rows<T>(n_rows, n_cols, {x, w, y, res, h_out}, {xs, ys, rs, hs}, FAT_NORM_FWD_BPS, FAT_NORM_FWD_PPT);
    if (p.fast) {
      FAT_VPT_SWITCH(p.vpt, (norm_fwd_kernel<T, W, VPT, true><<<p.grid, kThreads, 0, st>>>(
          (const T*)x, (const T*)w, (T*)y, mean, n_rows, int(n_cols), xs, ys, eps, p.G, (const T*)res, (T*)h_out, rs, hs)));
      return check_launch("add_norm_fwd");
    }
    if (int rc = add_rows_t<T>(x, res, h_out, n_rows, n_cols, xs, rs, hs, st)) return rc;
    x = h_out;
    xs = hs;
  }
  RowPlan p = plan_rows<T>(n_rows, n_cols, {x, w, y}, {xs, ys}, FAT_NORM_FWD_BPS, FAT_NORM_FWD_PPT);
  if (p.fast) {
    FAT_VPT_SWITCH(p.vpt, (norm_fwd_kernel<T, W, VPT><<<p.grid, kThreads, 0, st>>>(
        (const T*)x, (const T*)w, (T*)y, mean, n_rows, int(n_cols), xs, ys, eps, p.G)));
  } else {
    row_slow_kernel<T, kNormFwd><<<p.grid, kThreads, 0, st>>>((const T*)x, nullptr, (const T*)w, mean, nullptr,
                                                               (T*)y, nullptr, n_rows, n_cols, xs, 0, ys, eps);
  }
  return check_launch("norm_fwd");
}

template <typename T>
int norm_bwd_t(const void* d_out, const void* x, const void* w, const float* mean, void* d_x, void* d_w,
               void* ws, size_t ws_bytes, int64_t n_rows, int64_t n_cols, int64_t dos, int64_t xs, int64_t dxs,
               double eps, cudaStream_t st, const void* d_add = nullptr, int64_t das = 0) {
  using C = typename Elem<T>::C;
  constexpr int W = 16 / sizeof(T);
  // wide rows run with 512-thread blocks so that a thread owns one or two packs of a row: the per-thread
  // state (weight, d_weight partials, the row and the prefetched next row) then fits in 64 registers
  constexpr int kWide = 512;
#ifndef FAT_NORM_BWD16_WIDE
#define FAT_NORM_BWD16_WIDE 0
#endif
  // (16-bit rows of up to 2 x 256 packs go to the packed-arithmetic kernel, which keeps 256-thread blocks: two of them
  //  share an SM and fill each other's reduction barriers)
  const bool wide = n_cols / W > kThreads && !(sizeof(T) == 2 && n_cols / W <= 2 * kThreads && !FAT_NORM_BWD16_WIDE);
  const int threads = wide ? kWide : kThreads;
  RowPlan p = plan_rows<T>(n_rows, n_cols, {d_out, x, w, d_x, d_add}, {dos, xs, dxs, das}, FAT_NORM_BWD_BPS, FAT_NORM_BWD_PPT, threads);
  if (p.grid > norm_bwd_max_blocks()) p.grid = norm_bwd_max_blocks();
  if (size_t(p.grid) * size_t(n_cols) * sizeof(C) > ws_bytes) {
    set_error("norm_bwd: workspace of %zu bytes is smaller than the %zu needed", ws_bytes,
              size_t(p.grid) * size_t(n_cols) * sizeof(C));
    return FAT_ERR_WORKSPACE;
  }
  C* partial = reinterpret_cast<C*>(ws);
  if (p.fast) {
    auto go = [&](auto kern, size_t smem) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      kern<<<p.grid, threads, smem, st>>>((const T*)d_out, (const T*)x, (const T*)w, mean, (T*)d_x, partial,
                                         n_rows, int(n_cols), dos, xs, dxs, eps, p.G, (const T*)d_add, das);
    };
    bool launched16 = false;
    if constexpr (sizeof(T) == 2) {
      if (p.vpt <= 2) {                                     // 16-bit rows of up to two packs per thread: the packed-arithmetic kernel
        auto go16 = [&](auto kern, size_t smem) {
          if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
          kern<<<p.grid, threads, smem, st>>>((const T*)d_out, (const T*)x, (const T*)w, mean, (T*)d_x, partial,
                                             n_rows, int(n_cols), dos, xs, dxs, eps, p.G, (const T*)d_add, das);
        };
        const size_t smem1 = size_t(threads) * 1 * W * sizeof(float), smem2 = size_t(threads) * 2 * W * sizeof(float);
        if (d_add) {
          if (wide) { if (p.vpt == 1) go16(norm_bwd16_kernel<T, 1, kWide, true>, smem1); else go16(norm_bwd16_kernel<T, 2, kWide, true>, smem2); }
          else      { if (p.vpt == 1) go16(norm_bwd16_kernel<T, 1, kThreads, true>, smem1); else go16(norm_bwd16_kernel<T, 2, kThreads, true>, smem2); }
        } else {
          if (wide) { if (p.vpt == 1) go16(norm_bwd16_kernel<T, 1, kWide>, smem1); else go16(norm_bwd16_kernel<T, 2, kWide>, smem2); }
          else      { if (p.vpt == 1) go16(norm_bwd16_kernel<T, 1, kThreads>, smem1); else go16(norm_bwd16_kernel<T, 2, kThreads>, smem2); }
        }
        launched16 = true;
      }
    }
    if (launched16) {
    } else if (d_add) {
      if (wide) { FAT_VPT_SWITCH(p.vpt, go(norm_bwd_kernel<T, W, VPT, kWide, true>, size_t(kWide) * VPT * W * sizeof(C))); }
      else      { FAT_VPT_SWITCH(p.vpt, go(norm_bwd_kernel<T, W, VPT, kThreads, true>, size_t(kThreads) * VPT * W * sizeof(C))); }
    } else {
      if (wide) { FAT_VPT_SWITCH(p.vpt, go(norm_bwd_kernel<T, W, VPT, kWide>, size_t(kWide) * VPT * W * sizeof(C))); }
      else      { FAT_VPT_SWITCH(p.vpt, go(norm_bwd_kernel<T, W, VPT, kThreads>, size_t(kThreads) * VPT * W * sizeof(C))); }
    }
  } else {
    row_slow_kernel<T, kNormBwd><<<p.grid, kThreads, 0, st>>>((const T*)x, (const T*)d_out, (const T*)w, nullptr, mean,
                                                               (T*)d_x, partial, n_rows, n_cols, xs, dos, dxs, eps);
  }
  int rc = check_launch("norm_bwd");
  if (rc) return rc;
  if (d_add && !p.fast) {                                   // the generic kernel wrote the plain gradient: add in a second pass
    if ((rc = add_rows_t<T>(d_x, d_add, d_x, n_rows, n_cols, dxs, das, dxs, st))) return rc;
  }
  norm_bwd_reduce_kernel<T><<<unsigned((n_cols + 31) / 32), 32 * kReduceSlices, 0, st>>>(partial, (T*)d_w, p.grid, int(n_cols));
  return check_launch("norm_bwd_reduce");
}

template <typename T>
int softmax_fwd_t(const void* x, void* pr, int64_t n_rows, int64_t n_cols, int64_t xs, int64_t ps, double eps,
                  cudaStream_t st) {
  constexpr int W = 16 / sizeof(T);
  RowPlan p = plan_rows<T>(n_rows, n_cols, {x, pr}, {xs, ps}, FAT_SOFTMAX_BPS, FAT_SOFTMAX_PPT);
  if (p.fast) {
    FAT_VPT_SWITCH(p.vpt, (softmax_fwd_kernel<T, W, VPT><<<p.grid, kThreads, 0, st>>>(
        (const T*)x, (T*)pr, n_rows, int(n_cols), xs, ps, eps, p.G)));
  } else {
    row_slow_kernel<T, kSoftmaxFwd><<<p.grid, kThreads, 0, st>>>((const T*)x, nullptr, nullptr, nullptr, nullptr,
                                                                  (T*)pr, nullptr, n_rows, n_cols, xs, 0, ps, eps);
  }
  return check_launch("softmax_fwd");
}

template <typename T>
int softmax_bwd_t(const void* d_out, const void* x, void* d_x, int64_t n_rows, int64_t n_cols, int64_t dos,
                  int64_t xs, int64_t dxs, double eps, cudaStream_t st) {
  constexpr int W = 16 / sizeof(T);
  RowPlan p = plan_rows<T>(n_rows, n_cols, {d_out, x, d_x}, {dos, xs, dxs}, FAT_SOFTMAX_BPS, FAT_SOFTMAX_PPT);
  if (p.fast) {
    FAT_VPT_SWITCH(p.vpt, (softmax_bwd_kernel<T, W, VPT><<<p.grid, kThreads, 0, st>>>(
        (const T*)d_out, (const T*)x, (T*)d_x, n_rows, int(n_cols), dos, xs, dxs, eps, p.G)));
  } else {
    row_slow_kernel<T, kSoftmaxBwd><<<p.grid, kThreads, 0, st>>>((const T*)x, (const T*)d_out, nullptr, nullptr, nullptr,
                                                                  (T*)d_x, nullptr, n_rows, n_cols, xs, dos, dxs, eps);
  }
  return check_launch("softmax_bwd");
}

#define FAT_DTYPE_SWITCH(dtype, ...)                                                    \
  switch (dtype) {                                                                      \
    case FAT_F32:  { using T = float;          return __VA_ARGS__; }                    \
    case FAT_BF16: { using T = __nv_bfloat16;  return __VA_ARGS__; }                    \
    case FAT_F16:  { using T = __half;         return __VA_ARGS__; }                    \
    case FAT_F64:  { using T = double;         return __VA_ARGS__; }                    \
    default: set_error("unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE;        \
  }

int check_2d(const char* what, int64_t n_rows, int64_t n_cols) {
  if (n_rows < 0 || n_cols <= 0 || n_cols > (int64_t(1) << 30)) {
    set_error("%s: bad shape [%lld, %lld]", what, (long long)n_rows, (long long)n_cols);
    return FAT_ERR_SHAPE;
  }
  return FAT_OK;
}

}  // namespace
}  // namespace fat

static __device__ __align__(256) unsigned char g_norm_bwd_scratch[fat::kStaticScratchBytes];

namespace fat {
namespace {

// Device address of g_norm_bwd_scratch on the current device.  In host code the array's name is
// only a handle, not a device pointer, so the address is asked for once per device (with that
// device current) and cached.
int static_scratch(void** out) {
  static std::mutex mu;
  static void* cached[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("norm_bwd_static: cannot identify the current device (%s)", cudaGetErrorString(e));
    return FAT_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_norm_bwd_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("norm_bwd_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return FAT_ERR_LAUNCH;
    }
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return FAT_OK;
}

}  // namespace
}  // namespace fat

using namespace fat;

extern "C" {

int fat_swiglu_fwd(const void* gate, const void* value, void* out, int64_t n_rows, int64_t n_cols,
                   int64_t gs, int64_t vs, int64_t os, int dtype, void* stream) {
  if (int rc = check_2d("swiglu_fwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!gate || !value || !out) { set_error("swiglu_fwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, swiglu_fwd_t<T>(gate, value, out, n_rows, n_cols, gs, vs, os, (cudaStream_t)stream));
}

int fat_swiglu_bwd(const void* d_out, const void* gate, const void* value, void* d_gate, void* d_value,
                   int64_t n_rows, int64_t n_cols, int64_t dos, int64_t gs, int64_t vs, int64_t dgs, int64_t dvs,
                   int dtype, void* stream) {
  if (int rc = check_2d("swiglu_bwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!d_out || !gate || !value || !d_gate || !d_value) { set_error("swiglu_bwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, swiglu_bwd_t<T>(d_out, gate, value, d_gate, d_value, n_rows, n_cols, dos, gs, vs, dgs, dvs,
                                          (cudaStream_t)stream));
}

int fat_norm_fwd(const void* x, const void* weight, void* y, float* mean, int64_t n_rows, int64_t n_cols,
                 int64_t xs, int64_t ys, double eps, int dtype, void* stream) {
  if (int rc = check_2d("norm_fwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!x || !weight || !y || !mean) { set_error("norm_fwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, norm_fwd_t<T>(x, weight, y, mean, n_rows, n_cols, xs, ys, eps, (cudaStream_t)stream));
}

int fat_add_norm_fwd(const void* x, const void* residual, const void* weight, void* h_out, void* y, float* mean,
                     int64_t n_rows, int64_t n_cols, int64_t xs, int64_t rs, int64_t hs, int64_t ys, double eps, int dtype,
                     void* stream) {
  if (int rc = check_2d("add_norm_fwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!x || !residual || !weight || !h_out || !y || !mean) { set_error("add_norm_fwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, norm_fwd_t<T>(x, weight, y, mean, n_rows, n_cols, xs, ys, eps, (cudaStream_t)stream, residual,
                                        h_out, rs, hs));
}

int fat_add_norm_bwd(const void* d_y, const void* d_h, const void* h, const void* weight, const float* mean, void* d_sum,
                     void* d_weight, void* workspace, size_t workspace_bytes, int64_t n_rows, int64_t n_cols,
                     int64_t dys, int64_t dhs, int64_t hs, int64_t dss, double eps, int dtype, void* stream) {
  if (int rc = check_2d("add_norm_bwd", n_rows, n_cols)) return rc;
  if (!d_weight || !weight) { set_error("add_norm_bwd: null pointer"); return FAT_ERR_NULL; }
  if (n_rows > 0 && (!d_y || !h || !mean || !d_sum)) { set_error("add_norm_bwd: null pointer"); return FAT_ERR_NULL; }
  if (!workspace) { set_error("add_norm_bwd: null workspace"); return FAT_ERR_WORKSPACE; }
  FAT_DTYPE_SWITCH(dtype, norm_bwd_t<T>(d_y, h, weight, mean, d_sum, d_weight, workspace, workspace_bytes, n_rows, n_cols,
                                        dys, hs, dss, eps, (cudaStream_t)stream, d_h, dhs));
}

size_t fat_norm_bwd_workspace_bytes(int64_t n_rows, int64_t n_cols, int dtype) {
  (void)n_rows;
  if (n_cols <= 0) return 0;
  return size_t(norm_bwd_max_blocks()) * size_t(n_cols) * (dtype == FAT_F64 ? 8 : 4);
}

int fat_norm_bwd(const void* d_out, const void* x, const void* weight, const float* mean, void* d_x, void* d_weight,
                 void* workspace, size_t workspace_bytes, int64_t n_rows, int64_t n_cols,
                 int64_t dos, int64_t xs, int64_t dxs, double eps, int dtype, void* stream) {
  if (int rc = check_2d("norm_bwd", n_rows, n_cols)) return rc;
  if (!d_weight || !weight) { set_error("norm_bwd: null pointer"); return FAT_ERR_NULL; }
  if (n_rows > 0 && (!d_out || !x || !mean || !d_x)) { set_error("norm_bwd: null pointer"); return FAT_ERR_NULL; }
  if (!workspace) { set_error("norm_bwd: null workspace"); return FAT_ERR_WORKSPACE; }
  FAT_DTYPE_SWITCH(dtype, norm_bwd_t<T>(d_out, x, weight, mean, d_x, d_weight, workspace, workspace_bytes, n_rows, n_cols,
                                        dos, xs, dxs, eps, (cudaStream_t)stream));
}

size_t fat_norm_bwd_static_capacity(void) { return kStaticScratchBytes; }

int fat_norm_bwd_static(const void* d_out, const void* x, const void* weight, const float* mean, void* d_x, void* d_weight,
                        int64_t n_rows, int64_t n_cols, int64_t dos, int64_t xs, int64_t dxs, double eps, int dtype,
                        void* stream) {
  if (int rc = check_2d("norm_bwd_static", n_rows, n_cols)) return rc;
  const size_t need = fat_norm_bwd_workspace_bytes(n_rows, n_cols, dtype);
  if (need > kStaticScratchBytes) {
    set_error("norm_bwd_static: %lld columns need %zu bytes of scratch, the built-in array holds %zu; "
              "use fat_norm_bwd with a caller-owned workspace", (long long)n_cols, need, kStaticScratchBytes);
    return FAT_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  return fat_norm_bwd(d_out, x, weight, mean, d_x, d_weight, scratch, kStaticScratchBytes, n_rows, n_cols, dos, xs, dxs,
                      eps, dtype, stream);
}

int fat_softmax_fwd(const void* x, void* p, int64_t n_rows, int64_t n_cols, int64_t xs, int64_t ps,
                    double eps, int dtype, void* stream) {
  if (int rc = check_2d("softmax_fwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!x || !p) { set_error("softmax_fwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, softmax_fwd_t<T>(x, p, n_rows, n_cols, xs, ps, eps, (cudaStream_t)stream));
}

int fat_softmax_bwd(const void* d_out, const void* x, void* d_x, int64_t n_rows, int64_t n_cols,
                    int64_t dos, int64_t xs, int64_t dxs, double eps, int dtype, void* stream) {
  if (int rc = check_2d("softmax_bwd", n_rows, n_cols)) return rc;
  if (n_rows == 0) return FAT_OK;
  if (!d_out || !x || !d_x) { set_error("softmax_bwd: null pointer"); return FAT_ERR_NULL; }
  FAT_DTYPE_SWITCH(dtype, softmax_bwd_t<T>(d_out, x, d_x, n_rows, n_cols, dos, xs, dxs, eps, (cudaStream_t)stream));
}

}  // extern "C"
