// Rational attention on the CUDA cores (fp32 accumulation): the path for float32 tensors
// (tensor cores cannot hold the 1e-5 bar in one pass), for head sizes the tcgen05 kernels
// do not cover, and the on-device cross-check of the tcgen05 path.
//
// Tiling: 64 queries x 64 keys per step, 256 threads as a 16x16 grid.  Thread (ty,tx) owns
// score rows {ty+16i} and score columns {tx+16j}; Q/K/V tiles live in shared memory as
// float with rows padded by 4 floats, so every 128-bit shared load is conflict free.
// Forward keeps a running sum of sigma^4 only (sigma^4 <= 1, nothing to rescale).  Backward
// is two kernels without atomics: a query-major one (Delta, d_q) and a key-major one
// (d_k, d_v), each recomputing the scores it needs.
#include "attn_common.cuh"

namespace fat {
namespace {

constexpr int BM = 64, BN = 64, NT = 256;
constexpr int LDP = BN + 4;

template <typename T, int DP>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const T* __restrict__ base,
                                          int64_t row_stride, int row0, int T_len, int D, bool vec) {
  constexpr int LD = DP + 4;
  constexpr int W = 16 / sizeof(T);
  if (vec) {
    constexpr int PPR = DP / W;
    for (int idx = threadIdx.x; idx < BM * PPR; idx += NT) {
      const int r = idx / PPR, c = (idx % PPR) * W, row = row0 + r;
      float vals[W];
      if (row < T_len && c < D) {
        load_pack_cached<T, W>(base + int64_t(row) * row_stride + c, vals);
      } else {
#pragma unroll
        for (int j = 0; j < W; ++j) vals[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < W; j += 4)
        *reinterpret_cast<float4*>(&dst[r * LD + c + j]) = make_float4(vals[j], vals[j + 1], vals[j + 2], vals[j + 3]);
    }
  } else {
    for (int idx = threadIdx.x; idx < BM * DP; idx += NT) {
      const int r = idx / DP, c = idx % DP, row = row0 + r;
      dst[r * LD + c] = (row < T_len && c < D) ? Elem<T>::to_c(base[int64_t(row) * row_stride + c]) : 0.f;
    }
  }
}

// acc[i][j] += sum_d A[ty+16i][d] * Bm[tx+16j][d]
template <int DP>
__device__ __forceinline__ void gemm_nt(float (&acc)[4][4], const float* __restrict__ A,
                                        const float* __restrict__ Bm, int ty, int tx) {
  constexpr int LD = DP + 4;
#pragma unroll 2
  for (int d = 0; d < DP; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(&A[(ty + 16 * i) * LD + d]);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(&Bm[(tx + 16 * j) * LD + d]);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

// Column ownership of the [64][DP] output tiles: thread tx owns VW consecutive columns in
// each of NCH chunks, chunk c starting at column c*16*VW.
template <int DP> struct OutCols {
  static constexpr int VW = DP >= 64 ? 4 : 2;
  static constexpr int NCH = DP / 16 / VW;
  static constexpr int N = DP / 16;
  static __device__ __forceinline__ int col(int tx, int c, int e) { return c * 16 * VW + tx * VW + e; }
};

// o[i][*] += sum_k P[ty+16i][k] * V[k][cols(tx)]     (P is [64][LDP], V is [64][DP+4])
template <int DP>
__device__ __forceinline__ void gemm_nn(float (&o)[4][DP / 16], const float* __restrict__ P,
                                        const float* __restrict__ V, int ty, int tx) {
  using OC = OutCols<DP>;
  constexpr int LD = DP + 4;
#pragma unroll 2
  for (int k = 0; k < BN; k += 4) {
    float4 p4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p4[i] = *reinterpret_cast<const float4*>(&P[(ty + 16 * i) * LDP + k]);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      float vv[OC::N];
#pragma unroll
      for (int c = 0; c < OC::NCH; ++c) {
        if constexpr (OC::VW == 4) {
          const float4 t = *reinterpret_cast<const float4*>(&V[(k + kk) * LD + OC::col(tx, c, 0)]);
          vv[c * 4 + 0] = t.x; vv[c * 4 + 1] = t.y; vv[c * 4 + 2] = t.z; vv[c * 4 + 3] = t.w;
        } else {
          const float2 t = *reinterpret_cast<const float2*>(&V[(k + kk) * LD + OC::col(tx, c, 0)]);
          vv[c * 2 + 0] = t.x; vv[c * 2 + 1] = t.y;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pv = kk == 0 ? p4[i].x : kk == 1 ? p4[i].y : kk == 2 ? p4[i].z : p4[i].w;
#pragma unroll
        for (int n = 0; n < OC::N; ++n) o[i][n] = fmaf(pv, vv[n], o[i][n]);
      }
    }
  }
}

// Writes o*mul to `base`; when `lo` is given also writes the rounding residual round(o*mul - stored).
template <typename T, int DP>
__device__ __forceinline__ void store_rows(T* __restrict__ base, int64_t row_stride, int row0, int T_len, int D,
                                           const float (&o)[4][DP / 16], const float (&mul)[4], int ty, int tx,
                                           T* __restrict__ lo = nullptr) {
  using OC = OutCols<DP>;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty + 16 * i;
    if (row >= T_len) continue;
#pragma unroll
    for (int c = 0; c < OC::NCH; ++c)
#pragma unroll
      for (int e = 0; e < OC::VW; ++e) {
        const int col = OC::col(tx, c, e);
        if (col < D) {
          const float val = o[i][c * OC::VW + e] * mul[i];
          const T hi = Elem<T>::from_c(val);
          base[int64_t(row) * row_stride + col] = hi;
          if (lo) lo[int64_t(row) * row_stride + col] = Elem<T>::from_c(val - Elem<T>::to_c(hi));
        }
      }
  }
}

struct Score { float f, k; };   // f = sigma^4, k = 2 sigma^3 r^2 (derivative of f w.r.t. the score)

__device__ __forceinline__ Score score_terms(float qk, float scale, float slope, int row, int col) {
  const float s = qk * scale - slope * fabsf(float(row - col));
  const float r = rcp1p_abs(s);
  const float sg = rsigmoid(s, r);
  const float s2 = sg * sg;
  return Score{s2 * s2, 2.f * s2 * sg * r * r};
}

// ------------------------------------------------------------------ forward
template <typename T, int DP>
__global__ void __launch_bounds__(NT) attn_fwd_simt_kernel(AttnParams p, bool vec) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = DP + 4;
  float* Qs = smem; float* Ks = Qs + BM * LD; float* Vs = Ks + BN * LD; float* Ps = Vs + BN * LD;
  const int b = blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;   // long rows first
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int q0 = qt * BM;
  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kb = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  T* ob = static_cast<T*>(p.out) + b * p.os[0] + h * p.os[1];
  const float slope = p.slopes[h];

  load_tile<T, DP>(Qs, qb, p.qs[2], q0, p.T, p.D, vec);
  float o[4][DP / 16] = {};
  float l[4] = {0.f, 0.f, 0.f, 0.f};
  const int n_kt = p.causal ? qt + 1 : (p.T + BN - 1) / BN;
  for (int kt = 0; kt < n_kt; ++kt) {
    const int k0 = kt * BN;
    load_tile<T, DP>(Ks, kb, p.ks[2], k0, p.T, p.D, vec);
    load_tile<T, DP>(Vs, vb, p.vs[2], k0, p.T, p.D, vec);
    __syncthreads();
    float acc[4][4] = {};
    gemm_nt<DP>(acc, Qs, Ks, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = q0 + ty + 16 * i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = k0 + tx + 16 * j;
        const bool live = col < p.T && row < p.T && (!p.causal || col <= row) && key_kept(p, b, col);
        const float f = live ? score_terms(acc[i][j], p.scale, slope, row, col).f : 0.f;
        l[i] += f;
        Ps[(ty + 16 * i) * LDP + tx + 16 * j] = f;
      }
    }
    __syncthreads();
    gemm_nn<DP>(o, Ps, Vs, ty, tx);
    __syncthreads();
  }
  float inv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int m = 8; m > 0; m >>= 1) l[i] += __shfl_xor_sync(0xffffffffu, l[i], m);
    inv[i] = 1.f / (l[i] + p.eps);
    const int row = q0 + ty + 16 * i;
    if (tx == 0 && row < p.T) p.L[(int64_t(b) * p.H + h) * p.T + row] = l[i];
  }
  T* olo = p.out_lo ? static_cast<T*>(p.out_lo) + b * p.os[0] + h * p.os[1] : nullptr;
  store_rows<T, DP>(ob, p.os[2], q0, p.T, p.D, o, inv, ty, tx, olo);
}

// ------------------------------------------------------------------ backward, query-major: Delta and d_q
template <typename T, int DP>
__global__ void __launch_bounds__(NT) attn_bwd_dq_simt_kernel(AttnParams p, bool vec) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = DP + 4;
  float* Qs = smem; float* dOs = Qs + BM * LD; float* Ks = dOs + BM * LD; float* Vs = Ks + BN * LD;
  float* dSs = Vs + BN * LD; float* rowInv = dSs + BM * LDP; float* rowD = rowInv + BM;
  const int b = blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = qt * BM;
  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kb = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const T* ob = static_cast<const T*>(p.out) + b * p.os[0] + h * p.os[1];
  const T* dob = static_cast<const T*>(p.d_out) + b * p.dos[0] + h * p.dos[1];
  T* dqb = static_cast<T*>(p.d_q) + b * p.dqs[0] + h * p.dqs[1];
  const int64_t stat0 = (int64_t(b) * p.H + h) * p.T;
  const float slope = p.slopes[h];

  load_tile<T, DP>(Qs, qb, p.qs[2], q0, p.T, p.D, vec);
  load_tile<T, DP>(dOs, dob, p.dos[2], q0, p.T, p.D, vec);
  load_tile<T, DP>(Ks, ob, p.os[2], q0, p.T, p.D, vec);          // the O tile, parked in the K buffer
  const bool has_lo = p.out_lo != nullptr;                        // and its rounding residual in the V buffer
  if (has_lo) load_tile<T, DP>(Vs, static_cast<const T*>(p.out_lo) + b * p.os[0] + h * p.os[1], p.os[2], q0, p.T, p.D, vec);
  __syncthreads();
  for (int r = warp * 8; r < warp * 8 + 8; ++r) {
    float s = 0.f;
    for (int d = lane; d < DP; d += 32) s = fmaf(dOs[r * LD + d], has_lo ? Ks[r * LD + d] + Vs[r * LD + d] : Ks[r * LD + d], s);
    s = warp_sum(s);
    if (lane == 0) {
      const int row = q0 + r;
      rowD[r] = s;
      rowInv[r] = row < p.T ? 1.f / (p.L[stat0 + row] + p.eps) : 0.f;
      if (row < p.T) p.delta[stat0 + row] = s;
    }
  }
  __syncthreads();

  float dq[4][DP / 16] = {};
  const int n_kt = p.causal ? qt + 1 : (p.T + BN - 1) / BN;
  for (int kt = 0; kt < n_kt; ++kt) {
    const int k0 = kt * BN;
    load_tile<T, DP>(Ks, kb, p.ks[2], k0, p.T, p.D, vec);
    load_tile<T, DP>(Vs, vb, p.vs[2], k0, p.T, p.D, vec);
    __syncthreads();
    float s[4][4] = {}, dp[4][4] = {};
    gemm_nt<DP>(s, Qs, Ks, ty, tx);
    gemm_nt<DP>(dp, dOs, Vs, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rl = ty + 16 * i, row = q0 + rl;
      const float dlt = rowD[rl], inv = rowInv[rl];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = k0 + tx + 16 * j;
        const bool live = col < p.T && row < p.T && (!p.causal || col <= row) && key_kept(p, b, col);
        dSs[rl * LDP + tx + 16 * j] =
            live ? score_terms(s[i][j], p.scale, slope, row, col).k * (dp[i][j] - dlt) * inv : 0.f;
      }
    }
    __syncthreads();
    gemm_nn<DP>(dq, dSs, Ks, ty, tx);
    __syncthreads();
  }
  const float mul[4] = {p.scale, p.scale, p.scale, p.scale};
  store_rows<T, DP>(dqb, p.dqs[2], q0, p.T, p.D, dq, mul, ty, tx);
}

// ------------------------------------------------------------------ backward, key-major: d_k and d_v
template <typename T, int DP>
__global__ void __launch_bounds__(NT) attn_bwd_dkv_simt_kernel(AttnParams p, bool vec) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = DP + 4;
  float* Ks = smem; float* Vs = Ks + BN * LD; float* Qs = Vs + BN * LD; float* dOs = Qs + BM * LD;
  float* PsT = dOs + BM * LD; float* dSsT = PsT + BN * LDP; float* rowInv = dSsT + BN * LDP; float* rowD = rowInv + BM;
  const int b = blockIdx.z, h = blockIdx.y, kt = blockIdx.x;                    // early key tiles are the long ones
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int k0 = kt * BN;
  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kb = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vb = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const T* dob = static_cast<const T*>(p.d_out) + b * p.dos[0] + h * p.dos[1];
  T* dkb = static_cast<T*>(p.d_k) + b * p.dks[0] + h * p.dks[1];
  T* dvb = static_cast<T*>(p.d_v) + b * p.dvs[0] + h * p.dvs[1];
  const int64_t stat0 = (int64_t(b) * p.H + h) * p.T;
  const float slope = p.slopes[h];

  load_tile<T, DP>(Ks, kb, p.ks[2], k0, p.T, p.D, vec);
  load_tile<T, DP>(Vs, vb, p.vs[2], k0, p.T, p.D, vec);
  float dk[4][DP / 16] = {}, dv[4][DP / 16] = {};
  const int n_qt = (p.T + BM - 1) / BM;
  for (int qt = p.causal ? kt : 0; qt < n_qt; ++qt) {
    const int q0 = qt * BM;
    load_tile<T, DP>(Qs, qb, p.qs[2], q0, p.T, p.D, vec);
    load_tile<T, DP>(dOs, dob, p.dos[2], q0, p.T, p.D, vec);
    if (threadIdx.x < BM) {
      const int row = q0 + threadIdx.x;
      rowInv[threadIdx.x] = row < p.T ? 1.f / (p.L[stat0 + row] + p.eps) : 0.f;
      rowD[threadIdx.x] = row < p.T ? p.delta[stat0 + row] : 0.f;
    }
    __syncthreads();
    float s[4][4] = {}, dp[4][4] = {};
    gemm_nt<DP>(s, Qs, Ks, ty, tx);
    gemm_nt<DP>(dp, dOs, Vs, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rl = ty + 16 * i, row = q0 + rl;
      const float dlt = rowD[rl], inv = rowInv[rl];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cl = tx + 16 * j, col = k0 + cl;
        const bool live = col < p.T && row < p.T && (!p.causal || col <= row) && key_kept(p, b, col);
        Score sc = score_terms(s[i][j], p.scale, slope, row, col);
        PsT[cl * LDP + rl] = live ? sc.f * inv : 0.f;
        dSsT[cl * LDP + rl] = live ? sc.k * (dp[i][j] - dlt) * inv : 0.f;
      }
    }
    __syncthreads();
    gemm_nn<DP>(dv, PsT, dOs, ty, tx);
    gemm_nn<DP>(dk, dSsT, Qs, ty, tx);
    __syncthreads();
  }
  const float one[4] = {1.f, 1.f, 1.f, 1.f};
  const float mul[4] = {p.scale, p.scale, p.scale, p.scale};
  store_rows<T, DP>(dvb, p.dvs[2], k0, p.T, p.D, dv, one, ty, tx);
  store_rows<T, DP>(dkb, p.dks[2], k0, p.T, p.D, dk, mul, ty, tx);
}

template <typename T>
bool tiles_vectorisable(const AttnParams& p, bool bwd) {
  constexpr int W = 16 / sizeof(T);
  if (p.D % W) return false;
  auto ok = [&](const void* ptr, const int64_t* s) {
    return aligned16(ptr) && s[0] % W == 0 && s[1] % W == 0 && s[2] % W == 0;
  };
  bool v = ok(p.q, p.qs) && ok(p.k, p.ks) && ok(p.v, p.vs);
  if (bwd) v = v && ok(p.out, p.os) && ok(p.d_out, p.dos);
  return v;
}

template <typename Kern>
int launch(Kern kern, const AttnParams& p, bool vec, int tiles, size_t smem, cudaStream_t st, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) { set_error("%s: cannot reserve %zu bytes of shared memory: %s", what, smem, cudaGetErrorString(e)); return FAT_ERR_LAUNCH; }
  dim3 grid(tiles, p.H, p.B);
  kern<<<grid, NT, smem, st>>>(p, vec);
  return check_launch(what);
}

template <typename T, int DP>
int fwd_t(const AttnParams& p, cudaStream_t st) {
  constexpr size_t smem = (size_t(3) * BM * (DP + 4) + BM * LDP) * sizeof(float);
  return launch(attn_fwd_simt_kernel<T, DP>, p, tiles_vectorisable<T>(p, false), (p.T + BM - 1) / BM, smem, st, "attn_fwd_simt");
}

template <typename T, int DP>
int bwd_t(const AttnParams& p, cudaStream_t st) {
  const bool vec = tiles_vectorisable<T>(p, true);
  const int tiles = (p.T + BM - 1) / BM;
  constexpr size_t smem_dq = (size_t(4) * BM * (DP + 4) + BM * LDP + 2 * BM) * sizeof(float);
  constexpr size_t smem_dkv = (size_t(4) * BM * (DP + 4) + 2 * BM * LDP + 2 * BM) * sizeof(float);
  if (int rc = launch(attn_bwd_dq_simt_kernel<T, DP>, p, vec, tiles, smem_dq, st, "attn_bwd_dq_simt")) return rc;
  return launch(attn_bwd_dkv_simt_kernel<T, DP>, p, vec, tiles, smem_dkv, st, "attn_bwd_dkv_simt");
}

template <typename T>
int dispatch_d(const AttnParams& p, bool bwd, cudaStream_t st) {
  if (p.D <= 32) return bwd ? bwd_t<T, 32>(p, st) : fwd_t<T, 32>(p, st);
  if (p.D <= 64) return bwd ? bwd_t<T, 64>(p, st) : fwd_t<T, 64>(p, st);
  if (p.D <= 128) return bwd ? bwd_t<T, 128>(p, st) : fwd_t<T, 128>(p, st);
  set_error("attention: head size %d is not supported (D <= 128)", p.D);
  return FAT_ERR_UNSUPPORTED;
}

int dispatch(const AttnParams& p, int dtype, bool bwd, cudaStream_t st) {
  switch (dtype) {
    case FAT_F32: return dispatch_d<float>(p, bwd, st);
    case FAT_BF16: return dispatch_d<__nv_bfloat16>(p, bwd, st);
    case FAT_F16: return dispatch_d<__half>(p, bwd, st);
    default: set_error("attention: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE;
  }
}

}  // namespace

int attn_fwd_simt(const AttnParams& p, int dtype, cudaStream_t st) { return dispatch(p, dtype, false, st); }
int attn_bwd_simt(const AttnParams& p, int dtype, cudaStream_t st) { return dispatch(p, dtype, true, st); }

}  // namespace fat
