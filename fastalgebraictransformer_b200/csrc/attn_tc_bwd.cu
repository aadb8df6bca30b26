// Causal rational attention backward on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Default: prepare (1), which also clears a float32 d_q accumulator, the fused key-major
// kernel (4) that produces d_k, d_v and adds its d_q contributions with TMA reduce-add, and a convert pass.
// Deterministic variant: three launches, no atomics, bit-reproducible:
//   1. prepare:  per query row  inv = 1/(L+eps) and Delta = dO . O  (two padded float32 arrays), max|dO| per
//                (batch, head), and for bfloat16 tensors float16 copies of q and k
//   2. d_q kernel, query-major (one 128-query tile per CTA, key tiles streamed):
//                S = Q K^T, dP = dO V^T -> dS = g inv (dP - Delta) (16-bit, packed into TMEM over dP)
//                -> dQ += dS K                      with F = sigma^4, g = 2 sigma^3 r^2
//   3. d_k/d_v kernel, key-major (one 128-key tile per CTA, query tiles streamed), transposed:
//                S^T = K Q^T, dP^T = V dO^T -> P^T = F inv, dS^T (TMEM) -> dV += P^T dO, dK += dS^T Q
// In both main kernels the element-wise work is split in two phases so that the tensor core
// never waits for it: phase A needs only the scores (sigma, F, g), phase B only dP'.
// Eight element-wise warps share a tile: warpgroup w owns score columns [64w, 64w+64).
#include <type_traits>

#include "attn_tc_common.cuh"

namespace fat {
namespace {

using namespace tc;
using namespace tcattn;

// Operand formats.  tcgen05.mma kind::f16 takes both operands of one MMA in ONE 16-bit format (an f16 A
// with a bf16 B is an illegal instruction).  P^T carries the tensor dtype (it multiplies dO).  dS / dS^T
// is always float16: rounded to bfloat16 (8 significand bits) it leaves a few elements in 10^4 of d_q and
// d_k outside the element-wise bar rel 2e-2 / abs 1e-2, with float16's 11 bits none.  Its partners in the
// d_q and d_k contractions (K and Q) therefore have to be float16 as well: for bfloat16 tensors the prepare
// pass writes float16 copies of q and k into the workspace (exact for magnitudes in [2^-14, 65504]; smaller
// ones round to multiples of 2^-24; magnitudes of 65536 and more are clamped to 65504 and reported in bit 29
// of the status word - the CUDA-core path takes such tensors), and the main kernels load those instead, so
// S = Q K^T is formed from the copies too.  V and dO are used as they are.
//
// Ranges.  dS is proportional to dO, whose magnitude is the caller's (loss scaling, tiny late-training
// gradients), so the prepare pass also finds max|dO| per (batch, head) and the kernels store
//     dS_stored = 4 (the "g8" units) * kDsScale * c * dS,   c = 2^-e with  max|dO| c  in [0.5, 1),
// undone exactly in the epilogue multipliers.  With |dS| <= 4 p |dO_i| |V_j - O_i| the stored value stays below
// 65504 unless |V_j - O_i| exceeds ~90/sqrt(D) times what it is for unit-normal V; the conversion saturates.
// P^T is stored as 16 sigma^4 (the "F16" units) times kOpScale/(L+eps): p <= 1, and the power of two keeps small p
// out of the float16 subnormals.
constexpr float kOpScale = 256.0f;
constexpr float kDsScale = 4.0f;         // fused and key-major kernels: dS_stored = 4 kDsScale c dS
constexpr float kDsScaleQ = 64.0f;       // query-major d_q kernel: dS_stored = 4 kDsScaleQ c (L+eps) dS (1/(L+eps) is applied to the rows of d_q afterwards)
constexpr int kStatusF16Range = 0x20000000;
// Bias of a key that the padding mask takes out, in the kernels where a thread owns a key: sigma(-1e6) = 2.5e-7, so its
// sigma^4 and its gradient factor vanish against every kept key's (the reference fills such scores with -1e4).
constexpr float kMaskedKeyBias = -1.0e6f;
// With a padding mask hundreds of queries can share a handful of keys with nearly equal weights; rounded to bfloat16's 8
// significand bits those weights leave d_v = P^T dO a few elements in 10^5 outside the 16-bit bar (the errors of one key's
// column no longer average out).  Masked bfloat16 launches therefore hand P^T to the d_v product as value + residual.
template <typename T> constexpr bool kMaskedHiLo = std::is_same<T, __nv_bfloat16>::value;
__device__ __forceinline__ uint32_t pack_residual(float p0, float p1, uint32_t packed_bf16) {
  return Pack16<__nv_bfloat16>::pack(p0 - __uint_as_float(packed_bf16 << 16), p1 - __uint_as_float(packed_bf16 & 0xffff0000u));
}

// c and 1/c from the bits of max|dO| (a float32 with the sign cleared)
__device__ __forceinline__ void dout_scale(uint32_t max_bits, float& c, float& rc) {
  const uint32_t E = min(max((max_bits >> 23) & 0xffu, 32u), 222u);    // zero / denormal / inf / NaN: any finite power of two
  c = __uint_as_float((253u - E) << 23);
  rc = __uint_as_float((E + 1u) << 23);
}

// two float32 -> packed float16, round to nearest even, overflow clamped to +-65504
__device__ __forceinline__ uint32_t pack_ds(float lo, float hi) {
  uint32_t y;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(hi), "f"(lo));
  return y;
}

// 8 bfloat16 -> 8 float16; `flag` collects whether a magnitude was 65536 or more (or not a number)
__device__ __forceinline__ uint4 bf16x8_to_f16x8(uint4 v, uint32_t& flag) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = w[i];
    flag |= ((x & 0x7fff7fffu) + 0x38803880u) & 0x80008000u;            // either half >= 0x4780 (65536.0)
    w[i] = pack_ds(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
  }
  return v;
}

constexpr int kEwGroups = 2;                          // element-wise warpgroups per CTA
constexpr int kEwThreads = 128 * kEwGroups;
constexpr int kColsPerGroup = BLK / kEwGroups;        // score columns owned by one warpgroup
constexpr int kChunks = kColsPerGroup / 32;           // 32-column chunks per thread and phase
constexpr int kTmaWarp = 4 * kEwGroups, kMmaWarp = kTmaWarp + 1;
constexpr int kBwdThreads = kEwThreads + 64;          // + one TMA producer warp + one MMA issuer warp
constexpr int kBwdStages = 2;
constexpr int kDqKStages = 3;

__host__ __device__ inline int64_t pad_rows(int T) { return int64_t((T + BLK - 1) / BLK) * BLK; }
// Head of the workspace: Delta [B,H,Tp], kOpScale/(L+eps) [B,H,Tp] (Tp = T rounded up to whole tiles), bits of max|dO| [B,H].
__host__ __device__ inline uint32_t* dmax_of(const AttnParams& p) {
  return reinterpret_cast<uint32_t*>(p.delta + 2 * int64_t(p.B) * p.H * pad_rows(p.T));
}

// ------------------------------------------------------------------------------------- 1. prepare
// One block = kPrepRows consecutive (padded) rows of one (batch, head): the only divisions are one 32-bit pair per
// block (the kernel is bound by instruction issue as much as by memory; per-row 64-bit divisions doubled its time).
#ifndef FAT_PREP_ROWS
#define FAT_PREP_ROWS 64
#define FAT_PREP_UNROLL 2
#endif
constexpr int kPrepRows = FAT_PREP_ROWS, kPrepUnroll = FAT_PREP_UNROLL;
template <typename T, int D>
__global__ void __launch_bounds__(256)
attn_bwd_prepare_kernel(const AttnParams p, float* __restrict__ inv_out, uint32_t* __restrict__ dmax,
                        float* __restrict__ dq_zero, __half* __restrict__ q16, __half* __restrict__ k16) {
  __shared__ uint32_t block_max;
  if (threadIdx.x == 0) block_max = 0;
  __syncthreads();
  float amax = 0.f;
  uint32_t out_of_range = 0;
  constexpr int LPR = D / 8;                      // lanes per row, 16 bytes each
  constexpr int RPW = 32 / LPR;                   // rows per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const int Tp = int(pad_rows(p.T));
  const unsigned chunks = unsigned(Tp / kPrepRows);
  const int bh = int(blockIdx.x / chunks), t0 = int(blockIdx.x % chunks) * kPrepRows;
  const int b = bh / p.H, h = bh % p.H;
  const T* ob = static_cast<const T*>(p.out) + b * p.os[0] + h * p.os[1] + l * 8;
  const T* lob = p.out_lo ? static_cast<const T*>(p.out_lo) + b * p.os[0] + h * p.os[1] + l * 8 : nullptr;
  const T* dob = static_cast<const T*>(p.d_out) + b * p.dos[0] + h * p.dos[1] + l * 8;
  const float* Lrow = p.L + int64_t(bh) * p.T;
  float* delta_row = p.delta + int64_t(bh) * Tp;
  float* inv_row = inv_out + int64_t(bh) * Tp;
  if (dq_zero) {                                  // clear this block's rows of the float32 d_q accumulator (dense [B,H,T,D])
    const int rows = min(kPrepRows, p.T - t0);
    float4* z = reinterpret_cast<float4*>(dq_zero + (int64_t(bh) * p.T + t0) * D);
    for (int i = threadIdx.x; i < rows * (D / 4); i += 256) __stcs(z + i, make_float4(0.f, 0.f, 0.f, 0.f));
  }
#pragma unroll (kPrepUnroll)
  for (int t = t0 + warp * RPW + sub; t < t0 + kPrepRows; t += 8 * RPW) {
    const bool live = t < p.T;
    float g[8] = {}, o[8] = {};
    if (live) {
      load_pack_cached<T, 8>(dob + int64_t(t) * p.dos[2], g);
      load_pack_cached<T, 8>(ob + int64_t(t) * p.os[2], o);
      if (lob) {
        float lo[8];
        load_pack_cached<T, 8>(lob + int64_t(t) * p.os[2], lo);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += lo[i];
      }
    }
    if (q16 && live) {                            // float16 copies of this row of q (and k) (dense [B,H,T,D])
      const uint4 qv = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + int64_t(t) * p.qs[2] + l * 8));
      const int64_t at = (int64_t(bh) * p.T + t) * D + l * 8;
      *reinterpret_cast<uint4*>(q16 + at) = bf16x8_to_f16x8(qv, out_of_range);
      if (k16) {                                  // (the fused kernel converts its K tile itself)
        const uint4 kv = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1] + int64_t(t) * p.ks[2] + l * 8));
        *reinterpret_cast<uint4*>(k16 + at) = bf16x8_to_f16x8(kv, out_of_range);
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dot = fmaf(g[i], o[i], dot); amax = fmaxf(amax, fabsf(g[i])); }
#pragma unroll
    for (int m = LPR / 2; m > 0; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
    if (l == 0) {                                 // rows in the padding get 0
      delta_row[t] = dot;
      inv_row[t] = live ? kOpScale / (Lrow[t] + p.eps) : 0.f;
    }
  }
  // max |dO| of this (batch, head): magnitudes compare like their bit patterns
  uint32_t mb = __float_as_uint(amax);
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, m));
  if (lane == 0) atomicMax(&block_max, mb);
  __syncthreads();
  if (threadIdx.x == 0) atomicMax(dmax + bh, block_max);
  if (out_of_range && p.status) atomicOr(p.status, kStatusF16Range);
}

// ------------------------------------------------------------------------------------- element-wise math
// Packed pair of raw score accumulators -> sigma-derived factors, in units that avoid every constant
// multiply: with s = acc*scale + bias, r = 1/(|s|+1), w = 1 + s r = 2 sigma,
//   g8  = w^3 r^2 = 8 sigma^3 r^2   (half of 8x the derivative of sigma^4; the constants go to the epilogues)
//   F16 = w^4     = 16 sigma^4      (when WANT_F)
template <bool WANT_F, bool SHARED>
__device__ __forceinline__ void score_fg2(f32x2 acc2, f32x2 scale2, f32x2 bias2, f32x2 one2, f32x2& F2, f32x2& g2) {
  const f32x2 s2 = fma2(acc2, scale2, bias2);
  f32x2 r2, w2;
  sigma_terms2<SHARED>(s2, one2, r2, w2);
  const f32x2 u2 = mul2(w2, r2);
  g2 = mul2(mul2(u2, u2), w2);
  if (WANT_F) { const f32x2 q2 = mul2(w2, w2); F2 = mul2(q2, q2); }
}

// TMEM column (relative to the start of a 128-column region) where warpgroup w keeps its packed
// 16-bit results: its elements live in the first half of the fp32 columns that only this warpgroup reads.
__device__ __forceinline__ uint32_t packed_col(int w, int chunk16) { return uint32_t(kColsPerGroup * w + 16 * chunk16); }

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Tile load that adds its bytes to a barrier whose expect_tx was posted separately.
template <int D>
__device__ __forceinline__ void load_tile_tma_noexpect(unsigned char* dst, const CUtensorMap* m, uint64_t* bar,
                                                       int row0, int h, int b) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_4d(dst + c * (BLK * 128), m, bar, c * 64, row0, h, b);
}

// Converts one thread's 32 fp32 values to 16-bit pairs and stores them into its row of a
// 128-byte-swizzled [128][D] staging tile, columns [col0, col0+32).
template <typename T>
__device__ __forceinline__ void stage_row32(unsigned char* stage, int r, int col0, const uint32_t (&v)[32], float mul) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = Pack16<T>::pack(__uint_as_float(v[2 * i]) * mul, __uint_as_float(v[2 * i + 1]) * mul);
#pragma unroll
  for (int sgm = 0; sgm < 4; ++sgm) {
    const int col = col0 + sgm * 8;
    *reinterpret_cast<uint4*>(stage + (col / 64) * (BLK * 128) + sw128_offset(r, (col % 64) / 8)) =
        make_uint4(w[4 * sgm], w[4 * sgm + 1], w[4 * sgm + 2], w[4 * sgm + 3]);
  }
}

// ------------------------------------------------------------------------------------- 2. d_q kernel
template <int D>
struct DqSmem {
  static constexpr int kTileBytes = BLK * D * 2;
  alignas(1024) unsigned char q[kTileBytes];               // reused as d_q staging in the epilogue
  alignas(1024) unsigned char dout[kTileBytes];
  alignas(1024) unsigned char k[kDqKStages][kTileBytes];   // K(j) is read by S(j) early and by dQ(j) late: three stages keep the loads ahead
  alignas(1024) unsigned char v[kBwdStages][kTileBytes];
  uint64_t qdo_full, k_full[kDqKStages], k_empty[kDqKStages], v_full[kBwdStages], v_empty[kBwdStages];
  uint64_t s_full, s_free, dp_full[2], ds_full[2], dq_full;   // dp_/ds_: one per dP buffer, so no barrier runs two phases ahead
  uint32_t tmem_base;
  int abort_flag;
};

struct DqMaps { CUtensorMap q, dout, k, v, dq; };

// TMEM columns: S [0,128)   dP / packed dS of even / odd key tiles [128,256) / [256,384)   dQ [384,384+D)
// dP is double-buffered: dP of the next key tile is computed while dS of the current one is still feeding dQ.
template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ DqMaps maps, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  using S = DqSmem<D>;
  S& sm = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  int rank, bh;
  if (!banded_tile((p.T + BLK - 1) / BLK, p.B * p.H, kBwdBands, rank, bh)) return;   // padding block of the banded order
  const int b = bh / p.H, h = bh % p.H;
  const int qt = (p.T + BLK - 1) / BLK - 1 - rank;           // long rows first
  const int n = p.causal ? qt + 1 : (p.T + BLK - 1) / BLK;   // key tiles 0..qt (causal) or all of them
  Guard g{&sm.abort_flag, p.status};

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.qdo_full, 1);
    mbar_init(&sm.s_full, 1); mbar_init(&sm.s_free, kEwThreads); mbar_init(&sm.dq_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&sm.dp_full[i], 1); mbar_init(&sm.ds_full[i], kEwThreads); }
    for (int i = 0; i < kDqKStages; ++i) { mbar_init(&sm.k_full[i], 1); mbar_init(&sm.k_empty[i], 1); }
    for (int i = 0; i < kBwdStages; ++i) { mbar_init(&sm.v_full[i], 1); mbar_init(&sm.v_empty[i], 1); }
    mbar_fence_init();
  }
  if (warp == kTmaWarp) { tmem_alloc(&sm.tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tS = tmem, tP0 = tmem + BLK, tQ = tmem + 3 * BLK;            // dP(j) lives at tP0 + (j & 1) * BLK
  float dscale, dscale_inv;                                  // c and 1/c of this (batch, head), see the top of the file
  dout_scale(dmax_of(p)[bh], dscale, dscale_inv);

  if (warp == kTmaWarp) {
    if (elect_one()) {
      mbar_expect_tx(&sm.qdo_full, 2 * S::kTileBytes);
      load_tile_tma_noexpect<D>(sm.q, &maps.q, &sm.qdo_full, qt * BLK, h, b);
      load_tile_tma_noexpect<D>(sm.dout, &maps.dout, &sm.qdo_full, qt * BLK, h, b);
      for (int j = 0; j < n; ++j) {
        const int ks = j % kDqKStages, vs = j % kBwdStages;
        if (!g.wait(&sm.k_empty[ks], ((j / kDqKStages) & 1) ^ 1, 40)) break;
        load_tile_tma<D>(sm.k[ks], &maps.k, &sm.k_full[ks], j * BLK, h, b);
        if (!g.wait(&sm.v_empty[vs], ((j / kBwdStages) & 1) ^ 1, 41)) break;
        load_tile_tma<D>(sm.v[vs], &maps.v, &sm.v_full[vs], j * BLK, h, b);
      }
    }
  } else if (warp == kMmaWarp) {
    if (elect_one()) {
      constexpr int H16 = Pack16<__half>::kFmt;
      constexpr uint32_t idesc_s = idesc_f16(BLK, BLK, H16, 0, 0);                  // S = Q K^T, float16 (q and k tiles are float16)
      constexpr uint32_t idesc_dp = idesc_f16(BLK, BLK, Pack16<T>::kFmt, 0, 0);     // dP = dO V^T, tensor dtype
      constexpr uint32_t idesc_dq = idesc_f16(BLK, D, H16, 0, 1);                   // dQ += dS K, float16
      const uint64_t qd = desc_kmajor(sm.q), dod = desc_kmajor(sm.dout);
      const uint64_t kd[kDqKStages] = {desc_kmajor(sm.k[0]), desc_kmajor(sm.k[1]), desc_kmajor(sm.k[2])};
      const uint64_t kd_mn[kDqKStages] = {desc_mnmajor(sm.k[0]), desc_mnmajor(sm.k[1]), desc_mnmajor(sm.k[2])};
      const uint64_t vd[kBwdStages] = {desc_kmajor(sm.v[0]), desc_kmajor(sm.v[1])};
      bool ok = g.wait(&sm.qdo_full, 0, 50) && g.wait(&sm.k_full[0], 0, 51);
      if (ok) { tc_fence_after(); issue_gemm_nt<D>(tS, qd, kd[0], idesc_s); mma_commit(&sm.s_full); }
      ok = ok && g.wait(&sm.v_full[0], 0, 52);
      if (ok) { tc_fence_after(); issue_gemm_nt<D>(tP0, dod, vd[0], idesc_dp); mma_commit(&sm.dp_full[0]); mma_commit(&sm.v_empty[0]); }
      for (int j = 0; j < n && ok; ++j) {
        const int ks = j % kDqKStages, ks1 = (j + 1) % kDqKStages, vs1 = (j + 1) % kBwdStages;
        const uint32_t kph1 = ((j + 1) / kDqKStages) & 1, vph1 = ((j + 1) / kBwdStages) & 1;
        if (j + 1 < n) {
          // S(j+1) as soon as phase A has read S(j); dP(j+1) into the other dP buffer (its previous tenant dS(j-1)
          // was consumed by dQ(j-1), issued before this point), so phase B of the next tile never waits for it
          if (!(ok = g.wait(&sm.s_free, j & 1, 53))) break;
          if (!(ok = g.wait(&sm.k_full[ks1], kph1, 54))) break;
          tc_fence_after();
          issue_gemm_nt<D>(tS, qd, kd[ks1], idesc_s);
          mma_commit(&sm.s_full);
          if (!(ok = g.wait(&sm.v_full[vs1], vph1, 56))) break;
          tc_fence_after();
          issue_gemm_nt<D>(tP0 + ((j + 1) & 1) * BLK, dod, vd[vs1], idesc_dp);
          mma_commit(&sm.dp_full[(j + 1) & 1]);
          mma_commit(&sm.v_empty[vs1]);
        }
        if (!(ok = g.wait(&sm.ds_full[j & 1], (j >> 1) & 1, 55))) break;
        tc_fence_after();
        issue_gemm_tn<kColsPerGroup>(tQ, tP0 + (j & 1) * BLK, kd_mn[ks], idesc_dq, j > 0);       // dQ += dS K
        mma_commit(&sm.k_empty[ks]);
      }
      if (ok) mma_commit(&sm.dq_full);
    }
  } else {
    const int w = warp >> 2;                                 // column slice of this warpgroup
    const int r = tid & (BLK - 1);                           // query row inside the tile == TMEM lane
    const int row = qt * BLK + r;
    const uint32_t lane_base = uint32_t(warp & 3) * 32;
    const float slope = p.slopes[h], scale = p.scale;
    const int64_t srow = (int64_t(b) * p.H + h) * pad_rows(p.T) + row;
    const float dlt = p.delta[srow];                                               // Delta of this query
    const float ginv = p.delta[int64_t(p.B) * p.H * pad_rows(p.T) + srow] ;              // kOpScale/(L+eps)
    const f32x2 scale2 = pk2(scale, scale), half2 = pk2(1.0f, 1.0f);
    const float cs = kDsScaleQ * dscale;                     // dS_stored = g8 cs (dP - Delta)
    const f32x2 cs2 = pk2(cs, cs), ndlt2 = pk2(-dlt * cs, -dlt * cs);
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      f32x2 gq[kColsPerGroup / 2];
      // ---- phase A: g = sigma^3 r^2 / (L+eps) from the scores
      if (!(ok = g.wait(&sm.s_full, j & 1, 60))) break;
      tc_fence_after();
      // bias of key column c of this tile: -slope |row - (j BLK + c)| = sl * c + base with sl = slope for keys up to the
      // query, -slope for keys after it (non-causal only); the diagonal tile of a non-causal problem takes the absolute
      // value element by element (ABS)
      const float sl = (!p.causal && j > qt) ? -slope : slope;
      const float base = sl * float(j * BLK - row);
      const f32x2 step2 = pk2(2.f * sl, 2.f * sl);
      // KM: a padding mask over the keys is in force (one 32-bit word per chunk, bit set = the key takes part)
      const uint32_t* keep_words = p.key_mask ? p.key_mask + int64_t(b) * p.mask_words + j * (BLK / 32) : nullptr;
      auto phase_a = [&](auto ABS, auto KM) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t sreg[32];
          tmem_ld32(tmem_addr(tS, lane_base, kColsPerGroup * w + 32 * c), sreg);
          const int col0 = kColsPerGroup * w + 32 * c;
          uint32_t keep = 0xffffffffu;
          if constexpr (decltype(KM)::value) keep = __ldg(keep_words + (col0 >> 5));
          tmem_wait_ld_regs(sreg);
          f32x2 bias2 = pk2(fmaf(sl, float(col0), base), fmaf(sl, float(col0 + 1), base));
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            f32x2 F2, g2, b2 = bias2;
            if constexpr (decltype(ABS)::value) {
              float b0, b1;
              upk2(bias2, b0, b1);
              b2 = pk2(-fabsf(b0), -fabsf(b1));
            }
            const f32x2 acc2 = pk2(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1]));
            if (rcp_shared(i, FAT_RCP_SHARE_BWD)) score_fg2<false, true>(acc2, scale2, b2, half2, F2, g2);
            else            score_fg2<false, false>(acc2, scale2, b2, half2, F2, g2);
            bias2 = add2(bias2, step2);
            if constexpr (decltype(KM)::value) {
              float g0, g1;
              upk2(g2, g0, g1);
              if (!(keep & (1u << (2 * i)))) g0 = 0.f;
              if (!(keep & (2u << (2 * i)))) g1 = 0.f;
              g2 = pk2(g0, g1);
            }
            gq[16 * c + i] = g2;
          }
        }
      };
      const bool abs_tile = !p.causal && j == qt;
      if (keep_words) { if (abs_tile) phase_a(std::true_type{}, std::true_type{}); else phase_a(std::false_type{}, std::true_type{}); }
      else            { if (abs_tile) phase_a(std::true_type{}, std::false_type{}); else phase_a(std::false_type{}, std::false_type{}); }
      tc_fence_before();
      mbar_arrive(&sm.s_free);
      // ---- phase B: dS = g (dP - Delta), packed over dP
      if (!(ok = g.wait(&sm.dp_full[j & 1], (j >> 1) & 1, 61))) break;
      tc_fence_after();
      const bool diag = p.causal && (j == qt);               // (non-causal: nothing is masked)
      const uint32_t tP = tP0 + (j & 1) * BLK;
      // (the diagonal tile gets its own copy of the loop: a run-time test inside the unrolled body would split it
      //  into basic blocks and keep the compiler from interleaving the independent pairs)
      auto phase_b = [&](auto DIAG) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t dreg[32], preg[16];
          tmem_ld32(tmem_addr(tP, lane_base, kColsPerGroup * w + 32 * c), dreg);
          tmem_wait_ld_regs(dreg);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const f32x2 ds2 = mul2(gq[16 * c + i], fma2(pk2(__uint_as_float(dreg[2 * i]), __uint_as_float(dreg[2 * i + 1])), cs2, ndlt2));
            float d0, d1;
            upk2(ds2, d0, d1);
            if constexpr (decltype(DIAG)::value) {
              if (kColsPerGroup * w + 32 * c + 2 * i > r) d0 = 0.f;
              if (kColsPerGroup * w + 32 * c + 2 * i + 1 > r) d1 = 0.f;
            }
            preg[i] = pack_ds(d0, d1);
          }
          tmem_st16(tmem_addr(tP, lane_base, packed_col(w, c)), preg);
        }
      };
      if (diag) phase_b(std::true_type{}); else phase_b(std::false_type{});
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.ds_full[j & 1]);
    }
    if (ok) ok = g.wait(&sm.dq_full, 0, 62);
    named_barrier(1, kEwThreads);
    if (!g.aborted()) {
      tc_fence_after();
      const float mul = 0.25f * scale * (ginv / kOpScale) * dscale_inv / kDsScaleQ;   // 2 (derivative) / 8 (g8 units) * scale / (L+eps), operand scale undone
      for (int col0 = 32 * w; col0 < D; col0 += 32 * kEwGroups) {   // warpgroups interleave 32-column chunks of d_q
        uint32_t oreg[32];
        tmem_ld32(tmem_addr(tQ, lane_base, col0), oreg);
        tmem_wait_ld_regs(oreg);
        stage_row32<T>(sm.q, r, col0, oreg, mul);
      }
      fence_async_smem();
      named_barrier(1, kEwThreads);
      if (tid == 0) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_store_4d(&maps.dq, sm.q + c * (BLK * 128), c * 64, qt * BLK, h, b);
        tma_store_commit();
        tma_store_wait_all();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------- 3. d_k / d_v kernel
template <int D>
struct DkvSmem {
  static constexpr int kTileBytes = BLK * D * 2;
  alignas(1024) unsigned char k[kTileBytes];
  alignas(1024) unsigned char v[kTileBytes];
  alignas(1024) unsigned char q[kBwdStages][kTileBytes];     // reused as d_v / d_k staging in the epilogue
  alignas(1024) unsigned char dout[kBwdStages][kTileBytes];
  alignas(16) float delta[kBwdStages][BLK];                  // Delta and 1/(L+eps) of the staged query tile
  alignas(16) float inv[kBwdStages][BLK];
  uint64_t kv_full, q_full[kBwdStages], q_empty[kBwdStages], do_full[kBwdStages], do_empty[kBwdStages];
  uint64_t s_full, p_full, dp_full, ds_full, acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct DkvMaps { CUtensorMap q, dout, k, v, dk, dv; };

// TMEM columns: S^T / packed P^T [0,128)   dP'^T / packed dS^T [128,256)   dV [256,256+D)   dK [256+D,256+2D)
// MASKED: a padding mask over the keys is in force (p.key_mask is set).  A separate instantiation, so that the kernel of
// the unmasked case carries none of it.
template <typename T, int D, bool MASKED>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ DkvMaps maps, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  using S = DkvSmem<D>;
  S& sm = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  int kt, bh;                                                // rank = key tile: early key tiles see the most queries
  if (!banded_tile((p.T + BLK - 1) / BLK, p.B * p.H, kBwdBands, kt, bh)) return;     // padding block of the banded order
  const int b = bh / p.H, h = bh % p.H;
  const int n_q_total = (p.T + BLK - 1) / BLK;
  const int q0 = p.causal ? kt : 0;                          // first query tile that sees this key tile
  const int n = n_q_total - q0;                              // query tiles q0..n_q_total-1
  Guard g{&sm.abort_flag, p.status};

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.kv_full, 1); mbar_init(&sm.s_full, 1); mbar_init(&sm.p_full, kEwThreads);
    mbar_init(&sm.dp_full, 1); mbar_init(&sm.ds_full, kEwThreads); mbar_init(&sm.acc_full, 1);
    for (int i = 0; i < kBwdStages; ++i) {
      mbar_init(&sm.q_full[i], 1); mbar_init(&sm.q_empty[i], 1); mbar_init(&sm.do_full[i], 1); mbar_init(&sm.do_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == kTmaWarp) { tmem_alloc(&sm.tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tS = tmem, tP = tmem + BLK, tV = tmem + 2 * BLK, tK = tmem + 2 * BLK + D;
  float dscale, dscale_inv;                                  // c and 1/c of this (batch, head), see the top of the file
  dout_scale(dmax_of(p)[bh], dscale, dscale_inv);

  if (warp == kTmaWarp) {
    if (elect_one()) {
      mbar_expect_tx(&sm.kv_full, 2 * S::kTileBytes);
      load_tile_tma_noexpect<D>(sm.k, &maps.k, &sm.kv_full, kt * BLK, h, b);
      load_tile_tma_noexpect<D>(sm.v, &maps.v, &sm.kv_full, kt * BLK, h, b);
      const float* delta_bh = p.delta + (int64_t(b) * p.H + h) * pad_rows(p.T);
      const float* inv_bh = delta_bh + int64_t(p.B) * p.H * pad_rows(p.T);
      for (int it = 0; it < n; ++it) {
        const int st = it % kBwdStages, qi = q0 + it;
        const uint32_t ph = (it / kBwdStages) & 1;
        if (!g.wait(&sm.q_empty[st], ph ^ 1, 70)) break;
        mbar_expect_tx(&sm.q_full[st], S::kTileBytes + 2 * BLK * 4);
        load_tile_tma_noexpect<D>(sm.q[st], &maps.q, &sm.q_full[st], qi * BLK, h, b);
        bulk_load(sm.delta[st], delta_bh + qi * BLK, BLK * 4, &sm.q_full[st]);
        bulk_load(sm.inv[st], inv_bh + qi * BLK, BLK * 4, &sm.q_full[st]);
        if (!g.wait(&sm.do_empty[st], ph ^ 1, 71)) break;
        load_tile_tma<D>(sm.dout[st], &maps.dout, &sm.do_full[st], qi * BLK, h, b);
      }
    }
  } else if (warp == kMmaWarp) {
    if (elect_one()) {
      constexpr int F = Pack16<T>::kFmt, H16 = Pack16<__half>::kFmt;
      constexpr uint32_t idesc_s = idesc_f16(BLK, BLK, H16, 0, 0);       // S^T = K Q^T, float16 (q and k tiles are float16)
      constexpr uint32_t idesc_dp = idesc_f16(BLK, BLK, F, 0, 0);        // dP^T = V dO^T, tensor dtype
      constexpr uint32_t idesc_dv = idesc_f16(BLK, D, F, 0, 1);          // dV += P^T dO, tensor dtype
      constexpr uint32_t idesc_dk = idesc_f16(BLK, D, H16, 0, 1);        // dK += dS^T Q, float16
      const uint64_t kd = desc_kmajor(sm.k), vd = desc_kmajor(sm.v);
      const uint64_t qd[kBwdStages] = {desc_kmajor(sm.q[0]), desc_kmajor(sm.q[1])};
      const uint64_t qd_mn[kBwdStages] = {desc_mnmajor(sm.q[0]), desc_mnmajor(sm.q[1])};
      const uint64_t dod[kBwdStages] = {desc_kmajor(sm.dout[0]), desc_kmajor(sm.dout[1])};
      const uint64_t dod_mn[kBwdStages] = {desc_mnmajor(sm.dout[0]), desc_mnmajor(sm.dout[1])};
      bool ok = g.wait(&sm.kv_full, 0, 80) && g.wait(&sm.q_full[0], 0, 81);
      if (ok) { tc_fence_after(); issue_gemm_nt<D>(tS, kd, qd[0], idesc_s); mma_commit(&sm.s_full); }
      ok = ok && g.wait(&sm.do_full[0], 0, 82);
      if (ok) { tc_fence_after(); issue_gemm_nt<D>(tP, vd, dod[0], idesc_dp); mma_commit(&sm.dp_full); }
      for (int it = 0; it < n && ok; ++it) {
        const int st = it % kBwdStages, st1 = (it + 1) % kBwdStages;
        const uint32_t ph1 = ((it + 1) / kBwdStages) & 1;
        if (!(ok = g.wait(&sm.p_full, it & 1, 83))) break;
        tc_fence_after();
        if constexpr (MASKED && kMaskedHiLo<T>) issue_gemm_tn_hilo(tV, tS, dod_mn[st], idesc_dv, it > 0);
        else issue_gemm_tn<kColsPerGroup>(tV, tS, dod_mn[st], idesc_dv, it > 0);      // dV += P^T dO
        mma_commit(&sm.do_empty[st]);
        if (it + 1 < n) {
          if (!(ok = g.wait(&sm.q_full[st1], ph1, 84))) break;
          tc_fence_after();
          issue_gemm_nt<D>(tS, kd, qd[st1], idesc_s);        // S^T of the next query tile
          mma_commit(&sm.s_full);
        }
        if (!(ok = g.wait(&sm.ds_full, it & 1, 85))) break;
        tc_fence_after();
        issue_gemm_tn<kColsPerGroup>(tK, tP, qd_mn[st], idesc_dk, it > 0);       // dK += dS^T Q
        mma_commit(&sm.q_empty[st]);
        if (it + 1 < n) {
          if (!(ok = g.wait(&sm.do_full[st1], ph1, 86))) break;
          tc_fence_after();
          issue_gemm_nt<D>(tP, vd, dod[st1], idesc_dp);      // dP^T of the next query tile
          mma_commit(&sm.dp_full);
        }
      }
      if (ok) mma_commit(&sm.acc_full);
    }
  } else {
    const int w = warp >> 2;                                 // query-column slice of this warpgroup
    const int r = tid & (BLK - 1);                           // key row inside the tile == TMEM lane
    const int key = kt * BLK + r;
    const bool kept = !MASKED || key >= p.T || key_kept(p, b, key);     // a key the padding mask takes out gets a bias that zeroes it
    constexpr bool hilo = MASKED && kMaskedHiLo<T>;
    const uint32_t lane_base = uint32_t(warp & 3) * 32;
    const float slope = p.slopes[h], scale = p.scale;
    const f32x2 scale2 = pk2(scale, scale), half2 = pk2(1.0f, 1.0f);
    const float cs = kDsScale * dscale / kOpScale;           // dS_stored = g8 (kOpScale/(L+eps)) cs (dP - Delta)
    const f32x2 cs2 = pk2(cs, cs);
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int st = it % kBwdStages, qi = q0 + it;
      const bool diag = (qi == kt);
      f32x2 gq[kColsPerGroup / 2];
      // ---- phase A: p = sigma^4 / (L+eps) -> packed P^T over S^T; g / (L+eps) kept in registers
      if (!(ok = g.wait(&sm.q_full[st], (it / kBwdStages) & 1, 93))) break;       // Delta / inv arrived with the Q tile
      if (!(ok = g.wait(&sm.s_full, it & 1, 90))) break;
      tc_fence_after();
      // bias of query column c: -slope |key - (qi BLK + c)| = -sl * c + base with sl = slope for queries from the key on,
      // -slope for queries before it (non-causal only); MODE 1: causal diagonal tile (queries before the key are masked),
      // MODE 2: non-causal diagonal tile (absolute value element by element, nothing masked)
      const float sl = (!p.causal && qi < kt) ? -slope : slope;
      const float base = (!MASKED || kept) ? sl * float(key - qi * BLK) : kMaskedKeyBias;
      const f32x2 step2 = pk2(-2.f * sl, -2.f * sl);
      const float* iv = sm.inv[st];
      auto phase_a = [&](auto MODE, auto HL) { // the diagonal tile gets its own copy (no run-time test in the unrolled body)
        constexpr int kMode = decltype(MODE)::value;
        constexpr bool kHiLo = decltype(HL)::value && std::is_same<T, __nv_bfloat16>::value;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t sreg[32], preg[16], lreg[kHiLo ? 16 : 1];
          tmem_ld32(tmem_addr(tS, lane_base, kColsPerGroup * w + 32 * c), sreg);
          tmem_wait_ld_regs(sreg);
          const int col0 = kColsPerGroup * w + 32 * c;
          f32x2 bias2 = pk2(fmaf(-sl, float(col0), base), fmaf(-sl, float(col0 + 1), base));
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 iv2f = *reinterpret_cast<const float2*>(iv + col0 + 2 * i);
            const f32x2 iv2 = pk2(iv2f.x, iv2f.y);
            f32x2 F2, g2, b2 = bias2;
            if constexpr (kMode == 2) {
              float b0, b1;
              upk2(bias2, b0, b1);
              b2 = pk2(-fabsf(b0), -fabsf(b1));
            }
            const f32x2 acc2 = pk2(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1]));
            if (rcp_shared(i, FAT_RCP_SHARE_BWD)) score_fg2<true, true>(acc2, scale2, b2, half2, F2, g2);
            else                                  score_fg2<true, false>(acc2, scale2, b2, half2, F2, g2);
            bias2 = add2(bias2, step2);
            F2 = mul2(F2, iv2);
            g2 = mul2(g2, iv2);
            float p0, p1;
            upk2(F2, p0, p1);
            if constexpr (kMode == 1) {                       // queries before the key see nothing of it
              float g0, g1;
              upk2(g2, g0, g1);
              if (col0 + 2 * i < r) { p0 = 0.f; g0 = 0.f; }
              if (col0 + 2 * i + 1 < r) { p1 = 0.f; g1 = 0.f; }
              g2 = pk2(g0, g1);
            }
            gq[16 * c + i] = g2;
            preg[i] = Pack16<T>::pack(p0, p1);
            if constexpr (kHiLo) lreg[i] = pack_residual(p0, p1, preg[i]);
          }
          if constexpr (kHiLo) {
            tmem_st16(tmem_addr(tS, lane_base, col0), preg);
            tmem_st16(tmem_addr(tS, lane_base, col0 + 16), lreg);
          } else {
            tmem_st16(tmem_addr(tS, lane_base, packed_col(w, c)), preg);
          }
        }
      };
      if (!diag)         phase_a(std::integral_constant<int, 0>{}, std::integral_constant<bool, hilo>{});
      else if (p.causal) phase_a(std::integral_constant<int, 1>{}, std::integral_constant<bool, hilo>{});
      else               phase_a(std::integral_constant<int, 2>{}, std::integral_constant<bool, hilo>{});
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_full);
      // ---- phase B: dS^T = g (dP^T - Delta[q]) -> packed over dP^T
      if (!(ok = g.wait(&sm.dp_full, it & 1, 91))) break;
      tc_fence_after();
      const float* dl = sm.delta[st];
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        uint32_t dreg[32], preg[16];
        tmem_ld32(tmem_addr(tP, lane_base, kColsPerGroup * w + 32 * c), dreg);
        tmem_wait_ld_regs(dreg);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 d2 = *reinterpret_cast<const float2*>(dl + kColsPerGroup * w + 32 * c + 2 * i);
          const f32x2 ds2 = mul2(gq[16 * c + i], fma2(pk2(__uint_as_float(dreg[2 * i]), __uint_as_float(dreg[2 * i + 1])), cs2, pk2(-cs * d2.x, -cs * d2.y)));
          float d0, d1;
          upk2(ds2, d0, d1);
          preg[i] = pack_ds(d0, d1);
        }
        tmem_st16(tmem_addr(tP, lane_base, packed_col(w, c)), preg);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.ds_full);
    }
    if (ok) ok = g.wait(&sm.acc_full, 0, 92);
    named_barrier(1, kEwThreads);
    if (!g.aborted()) {
      // d_v (columns [0,D) of the accumulators) is staged in q[0], d_k (columns [D,2D)) in q[1]; the
      // warpgroups interleave 32-column chunks.  The multipliers undo the 16x (F16) and 8x (g8) units.
      tc_fence_after();
      for (int ch = w; ch < 2 * D / 32; ch += kEwGroups) {
        const bool is_dk = ch >= D / 32;
        const int col0 = (is_dk ? ch - D / 32 : ch) * 32;
        uint32_t oreg[32];
        tmem_ld32(tmem_addr(is_dk ? tK : tV, lane_base, col0), oreg);
        tmem_wait_ld_regs(oreg);
        stage_row32<T>(sm.q[is_dk ? 1 : 0], r, col0, oreg, is_dk ? 0.25f * scale * dscale_inv / kDsScale : 0.0625f / kOpScale);
      }
      fence_async_smem();
      named_barrier(1, kEwThreads);
      if (tid == 0) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_store_4d(&maps.dv, sm.q[0] + c * (BLK * 128), c * 64, kt * BLK, h, b);
          tma_store_4d(&maps.dk, sm.q[1] + c * (BLK * 128), c * 64, kt * BLK, h, b);
        }
        tma_store_commit();
        tma_store_wait_all();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tmem, kTmemCols);
}


// ------------------------------------------------------------------------------------- 4. fused d_k / d_v / d_q kernel
// Key-major: one CTA owns a 128-key tile and walks the 128-query tiles that see it.  With D = 128 every GEMM is a
// full 128x128x128 (tcgen05.mma below N = 128 runs at about half rate) and TMEM is exactly full:
//   R1 [0,128)    S^T, then the packed P^T over it         R2 [128,256)  dP^T, then dQ^T over it
//   dV [256,256+D)  dK [256+D,256+2D)
// dS^T goes to shared memory ([128 keys][128 queries], 16-bit): K-major A operand of dK += dS^T Q and MN-major B
// operand of dQ^T = K^T dS^T.  Four drain warps move dQ^T (head dimension on the TMEM lanes) through shared
// memory, transposed, into a float32 accumulator in global memory with TMA reduce-add, 32 query rows at a time.
// dO has a single buffer: dO(i+1) is only needed once dQ^T(i) has been drained, long after dV(i) released dO(i).
// The element-wise warps keep g for 64 score columns in registers between phase A and phase B, which needs
// about 168 registers per thread; the other warps need far fewer, so the warpgroups trade registers with
// setmaxnreg (the launch allocates 512 x 128).
constexpr int kFusedDrainWarp = 8, kFusedTmaWarp = 12, kFusedMmaWarpX = 13, kFusedMmaWarpY = 14, kFusedThreads = 512;
constexpr int kFusedRegsLaunch = 128, kFusedRegsEw = 168, kFusedRegsDrain = 104, kFusedRegsAux = 64;
static_assert(256 * kFusedRegsEw + 128 * kFusedRegsDrain + 128 * kFusedRegsAux <= kFusedThreads * kFusedRegsLaunch,
              "the warpgroups' register shares must fit in what the launch allocates");

template <int N> __device__ __forceinline__ void reg_share_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_share_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int D>
struct FusedSmem {
  static constexpr int kTileBytes = BLK * D * 2;
  alignas(1024) unsigned char k[kTileBytes];
  alignas(1024) unsigned char v[kTileBytes];
  alignas(1024) unsigned char q[2][kTileBytes];             // q[0] doubles as d_v staging in the epilogue
  alignas(1024) unsigned char dout[kTileBytes];             // doubles as d_k staging in the epilogue
  alignas(1024) unsigned char ds[BLK * BLK * 2];            // dS^T, 16-bit [128 keys][128 queries]
  alignas(1024) float dq_stage[64 * D];                     // d_q staging tile [64 query rows][D]
  alignas(16) float delta[2][BLK];
  alignas(16) float inv[2][BLK];
  uint64_t kv_full, q_full[2], q_empty[2], do_full, do_empty;
  uint64_t s_full, p_full, dp_full, ds_full, dq_full, dq_free, acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct FusedMaps { CUtensorMap q, dout, k, v, dk, dv, dq_acc; };    // dq_acc: float32, 32-row boxes

// MASKED: a padding mask over the keys is in force (p.key_mask is set).  A separate instantiation, so that the kernel of
// the unmasked case carries none of it.
template <typename T, int D, bool MASKED>
__global__ void __launch_bounds__(kFusedThreads, 1)
attn_bwd_fused_tc_kernel(const __grid_constant__ FusedMaps maps, const AttnParams p) {
  static_assert((D == 128 || D == 64) && kEwGroups == 2, "laid out for D = 64 or 128 and two element-wise warpgroups");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  using S = FusedSmem<D>;
  S& sm = *reinterpret_cast<S*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5;
  int kt, bh;                                                // rank = key tile: early key tiles see the most queries
  if (!banded_tile((p.T + BLK - 1) / BLK, p.B * p.H, kBwdBands, kt, bh)) return;     // padding block of the banded order
  const int b = bh / p.H, h = bh % p.H;
  const int n_q_total = (p.T + BLK - 1) / BLK;
  const int q0 = p.causal ? kt : 0;                          // first query tile that sees this key tile
  const int n = n_q_total - q0;                              // query tiles q0..n_q_total-1
  Guard g{&sm.abort_flag, p.status};
  if ((smem_u32(smem_raw) & 1023u) != 0) {                   // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0 && p.status) atomicOr(p.status, 0x40000000);
    return;                                                  // uniform: nobody has touched a barrier or TMEM yet
  }

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.kv_full, 1); mbar_init(&sm.s_full, 1); mbar_init(&sm.p_full, kEwThreads); mbar_init(&sm.dp_full, 1);
    mbar_init(&sm.ds_full, kEwThreads); mbar_init(&sm.dq_full, 1);
    mbar_init(&sm.dq_free, 128); mbar_init(&sm.acc_full, 2); mbar_init(&sm.do_full, 1); mbar_init(&sm.do_empty, 2);
    for (int i = 0; i < 2; ++i) { mbar_init(&sm.q_full[i], 1); mbar_init(&sm.q_empty[i], 1); }
    mbar_fence_init();
  }
  if (warp == kFusedTmaWarp) { tmem_alloc(&sm.tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tS = tmem, tP = tmem + BLK, tV = tmem + 2 * BLK, tK = tV + D;
  float dscale, dscale_inv;                                  // c and 1/c of this (batch, head), see the top of the file
  dout_scale(dmax_of(p)[bh], dscale, dscale_inv);

  // K and V of this CTA, and the first loads of the streamed tiles (both Q stages, dO), all issued before anything
  // else.  bfloat16 tensors: the whole CTA then turns the K tile into float16 in place before any role starts (four
  // 16-byte packs per thread, while the other loads are in flight; every K tile belongs to exactly one CTA, which
  // also checks its range).  Q tiles arrive as float16 from the copy the prepare pass made.
  const float* delta_bh = p.delta + (int64_t(b) * p.H + h) * pad_rows(p.T);
  const float* inv_bh = delta_bh + int64_t(p.B) * p.H * pad_rows(p.T);
  auto load_q = [&](int i) {                                  // Q tile, Delta and kOpScale/(L+eps) of query tile q0 + i
    const int st = i & 1, qi = q0 + i;
    mbar_expect_tx(&sm.q_full[st], S::kTileBytes + 2 * BLK * 4);
    load_tile_tma_noexpect<D>(sm.q[st], &maps.q, &sm.q_full[st], qi * BLK, h, b);
    bulk_load(sm.delta[st], delta_bh + qi * BLK, BLK * 4, &sm.q_full[st]);
    bulk_load(sm.inv[st], inv_bh + qi * BLK, BLK * 4, &sm.q_full[st]);
  };
  if (warp == kFusedTmaWarp && elect_one()) {
    mbar_expect_tx(&sm.kv_full, 2 * S::kTileBytes);
    load_tile_tma_noexpect<D>(sm.k, &maps.k, &sm.kv_full, kt * BLK, h, b);
    load_tile_tma_noexpect<D>(sm.v, &maps.v, &sm.kv_full, kt * BLK, h, b);
    load_q(0);
    load_tile_tma<D>(sm.dout, &maps.dout, &sm.do_full, q0 * BLK, h, b);
    if (n > 1) load_q(1);
  }
  if constexpr (!std::is_same<T, __half>::value) {
    if (g.wait(&sm.kv_full, 0, 139)) {
      uint32_t out_of_range = 0;
#pragma unroll
      for (int off = tid * 16; off < S::kTileBytes; off += kFusedThreads * 16)
        *reinterpret_cast<uint4*>(sm.k + off) = bf16x8_to_f16x8(*reinterpret_cast<const uint4*>(sm.k + off), out_of_range);
      if (out_of_range && p.status) atomicOr(p.status, kStatusF16Range);
      fence_async_smem();
    }
    __syncthreads();
  }

  if (warp >= kFusedTmaWarp) {
    reg_share_dec<kFusedRegsAux>();                             // warps 12..15 (15 only takes part in this)
    if (warp == kFusedTmaWarp) {
      // ---------------------------------------------------------------- TMA producer
      if (elect_one()) {
        for (int i = 1; i < n; ++i) {                                          // (Q(0), Q(1) and dO(0) are on their way)
          if (i >= 2) {
            if (!g.wait(&sm.q_empty[i & 1], ((i >> 1) & 1) ^ 1, 140)) break;
            load_q(i);
          }
          if (!g.wait(&sm.do_empty, (i & 1) ^ 1, 141)) break;                  // dV(i-1) and dP^T(i-1) have read dO(i-1)
          load_tile_tma<D>(sm.dout, &maps.dout, &sm.do_full, (q0 + i) * BLK, h, b);
        }
      }
    } else if (warp == kFusedMmaWarpX || warp == kFusedMmaWarpY) {
      // ---------------------------------------------------------------- tensor-core issuers
      if (elect_one()) {
        constexpr int F = Pack16<T>::kFmt, H16 = Pack16<__half>::kFmt;
        constexpr uint32_t idesc_s = idesc_f16(BLK, BLK, H16, 0, 0);        // S^T = K Q^T: both operands K-major, float16 (q and k tiles are float16)
        constexpr uint32_t idesc_dp = idesc_f16(BLK, BLK, F, 0, 0);         // dP^T = V dO^T: tensor dtype
        constexpr uint32_t idesc_dv = idesc_f16(BLK, D, F, 0, 1);           // dV += P^T dO: B (dO) MN-major, tensor dtype
        constexpr uint32_t idesc_dk = idesc_f16(BLK, D, H16, 0, 1);         // dK += dS^T Q: B (Q) MN-major, float16
        constexpr uint32_t idesc_dq = idesc_f16(BLK, BLK, H16, 1, 1);       // dQ^T: A = K (MN-major), B = dS^T (MN-major), float16
        bool ok = g.wait(&sm.kv_full, 0, 150);
        if (warp == kFusedMmaWarpX) {
          // ---- issuer X: dV as soon as P^T is written, then the next S^T into the same columns
          const uint64_t kd = desc_kmajor(sm.k);
          const uint64_t qd[2] = {desc_kmajor(sm.q[0]), desc_kmajor(sm.q[1])};
          const uint64_t dod_mn = desc_mnmajor(sm.dout);
          if (ok && (ok = g.wait(&sm.q_full[0], 0, 151))) {
            tc_fence_after();
            issue_gemm_nt<D>(tS, kd, qd[0], idesc_s);
            mma_commit(&sm.s_full);
          }
          for (int i = 0; i < n && ok; ++i) {
            const int st = i & 1, st1 = st ^ 1;
            // dO(i) and Q(i+1) were requested long ago: their barriers are settled before P^T, so that nothing but the issue
            // of the MMAs stands between the end of phase A and the next S^T (a satisfied wait still costs 150-250 cycles)
            if (!(ok = g.wait_polling(&sm.do_full, i & 1, 153))) break;
            if (i + 1 < n && !(ok = g.wait_polling(&sm.q_full[st1], ((i + 1) >> 1) & 1, 154))) break;
            if (!(ok = g.wait_polling(&sm.p_full, i & 1, 152))) break;
            tc_fence_after();
            if constexpr (MASKED && kMaskedHiLo<T>) issue_gemm_tn_hilo(tV, tS, dod_mn, idesc_dv, i > 0);
            else issue_gemm_tn<kColsPerGroup>(tV, tS, dod_mn, idesc_dv, i > 0);               // dV += P^T dO
            mma_commit(&sm.do_empty);                                                // X's share of releasing dO(i)
            if (i + 1 < n) {
              issue_gemm_nt<D>(tS, kd, qd[st1], idesc_s);                                // S^T of the next query tile
              mma_commit(&sm.s_full);
            }
          }
        } else {
          // ---- issuer Y: dQ^T and dK from the shared-memory dS^T tile, then the next dP^T once dQ^T has been drained
          const uint64_t vd = desc_kmajor(sm.v), kd_mn = desc_mnmajor(sm.k);
          const uint64_t dsd_k = desc_kmajor(sm.ds), dsd_mn = desc_mnmajor(sm.ds);
          const uint64_t qd_mn[2] = {desc_mnmajor(sm.q[0]), desc_mnmajor(sm.q[1])};
          const uint64_t dod = desc_kmajor(sm.dout);
          if (ok && (ok = g.wait(&sm.do_full, 0, 155))) {
            tc_fence_after();
            issue_gemm_nt<D>(tP, vd, dod, idesc_dp);
            mma_commit(&sm.dp_full);
            mma_commit(&sm.do_empty);
          }
          for (int i = 0; i < n && ok; ++i) {
            const int st = i & 1;
            if (!(ok = g.wait_polling(&sm.ds_full, i & 1, 156))) break;                  // phase B done: dS^T in smem, dP^T read
            tc_fence_after();
            // dQ^T = K^T dS^T over the keys.  The MMA is always 128 rows tall: with D = 64 the second 64-row chunk of the
            // MN-major A operand is the tile that follows K in shared memory (V), so TMEM lanes 64..127 receive numbers
            // nobody reads; the tensor pipe has the time, and M = 64 would use another accumulator layout.
#pragma unroll
            for (int s = 0; s < BLK / 16; ++s)
              mma_ss(tP, kd_mn + ((s * 2048) >> 4), dsd_mn + ((s * 2048) >> 4), idesc_dq, s > 0);
            mma_commit(&sm.dq_full);
#pragma unroll
            for (int s = 0; s < BLK / 16; ++s)                                           // dK += dS^T Q over the queries
              mma_ss(tK, dsd_k + ((((s / 4) * (BLK * 128) + (s % 4) * 32)) >> 4), qd_mn[st] + ((s * 2048) >> 4), idesc_dk, i > 0 || s > 0);
            mma_commit(&sm.q_empty[st]);
            if (i + 1 < n) {
              if (!(ok = g.wait_polling(&sm.do_full, (i + 1) & 1, 158))) break;         // (settled long before dQ^T is out)
              if (!(ok = g.wait_polling(&sm.dq_free, i & 1, 157))) break;                // dQ^T(i) has left TMEM
              tc_fence_after();
              issue_gemm_nt<D>(tP, vd, dod, idesc_dp);                                   // dP^T of the next query tile
              mma_commit(&sm.dp_full);
              mma_commit(&sm.do_empty);                                             // Y's share of releasing dO(i+1)
            }
          }
        }
        if (ok) mma_commit(&sm.acc_full);
      }
    }
  } else if (warp >= kFusedDrainWarp) {
    // ------------------------------------------------------------------ dQ^T drain: TMEM -> smem (transposed) -> reduce-add
    reg_share_dec<kFusedRegsDrain>();
    const int dl = tid - kFusedDrainWarp * 32;                   // head-dimension index == TMEM lane
    const uint32_t lane_base = uint32_t(warp & 3) * 32;
    float* stage0 = sm.dq_stage;                              // two staging tiles of [32 query rows][D] float32
    float* stage1 = sm.dq_stage + 32 * D;
    bool ok = true;
    // One quarter (32 query rows) of dQ^T: registers -> staging tile -> reduce-add.  One bulk group may still be reading
    // the other staging tile; the one that read this tile (the group before the newest) must be done before it is
    // overwritten, so every quarter commits exactly one group, issued or not.
    auto flush = [&](const uint32_t (&v)[32], float* stage, int row, bool wait_first) {
      if (wait_first) {
        if (dl == 0) tma_store_wait_read1();
        named_barrier(3, 128);
      }
      if (dl < D) {
#pragma unroll
        for (int qi = 0; qi < 32; ++qi) stage[qi * D + dl] = __uint_as_float(v[qi]);
      }
      fence_async_smem();
      named_barrier(3, 128);
      if (dl == 0) {
        if (row < p.T) tma_reduce_add_4d(&maps.dq_acc, stage, 0, row, h, b);
        tma_store_commit();                                   // also when nothing was issued (rows beyond T): the waits above count groups
      }
    };
    for (int i = 0; i < n; ++i) {
      const int row0 = (q0 + i) * BLK;
      if (!(ok = g.wait(&sm.dq_full, i & 1, 160))) break;
      tc_fence_after();
      uint32_t a[32], c[32];
      tmem_ld32(tmem_addr(tP, lane_base, 0), a);
      tmem_ld32(tmem_addr(tP, lane_base, 32), c);
      tmem_wait_ld_regs(a);
      tmem_wait_ld_regs(c);
      if (dl == 0) tma_store_wait_read();                     // both staging tiles are free (the previous step's reduces were issued long ago)
      named_barrier(3, 128);
      if (dl < D) {                                           // lanes beyond the head dimension hold nothing (D = 64)
#pragma unroll
        for (int qi = 0; qi < 32; ++qi) {
          stage0[qi * D + dl] = __uint_as_float(a[qi]);
          stage1[qi * D + dl] = __uint_as_float(c[qi]);
        }
      }
      tmem_ld32(tmem_addr(tP, lane_base, 64), a);            // second half into the same registers: dQ^T leaves TMEM early
      tmem_ld32(tmem_addr(tP, lane_base, 96), c);
      tmem_wait_ld_regs(a);
      tmem_wait_ld_regs(c);
      tc_fence_before();
      mbar_arrive(&sm.dq_free);                               // the next dP^T may be issued
      fence_async_smem();
      named_barrier(3, 128);
      if (dl == 0) {
        tma_reduce_add_4d(&maps.dq_acc, stage0, 0, row0, h, b);
        tma_store_commit();
        if (row0 + 32 < p.T) { tma_reduce_add_4d(&maps.dq_acc, stage1, 0, row0 + 32, h, b); }
        tma_store_commit();
      }
      flush(a, stage0, row0 + 64, true);                      // waits until only the stage1 group is still reading
      flush(c, stage1, row0 + 96, true);
    }
    if (dl == 0) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups
    reg_share_inc<kFusedRegsEw>();
    const int w = warp >> 2;                                 // query columns [64w, 64w+64) of each step
    const int r = tid & (BLK - 1);                           // key row inside the tile == TMEM lane
    const int key = kt * BLK + r;
    const bool kept = !MASKED || key >= p.T || key_kept(p, b, key);     // a key the padding mask takes out gets a bias that zeroes it
    constexpr bool hilo = MASKED && kMaskedHiLo<T>;
    const uint32_t lane_base = uint32_t(warp & 3) * 32;
    const float slope = p.slopes[h], scale = p.scale;
    const f32x2 scale2 = pk2(scale, scale), one2 = pk2(1.0f, 1.0f);
    const float cs = kDsScale * dscale / kOpScale;           // dS_stored = g8 (kOpScale/(L+eps)) cs (dP - Delta)
    const f32x2 cs2 = pk2(cs, cs);
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      const int st = i & 1, qi = q0 + i;
      const bool diag = (qi == kt);
      f32x2 gq[kColsPerGroup / 2];
      // ---- phase A: p = sigma^4 / (L+eps) -> packed P^T over S^T; g / (L+eps) kept in registers
      if (!(ok = g.wait(&sm.q_full[st], (i >> 1) & 1, 170))) break;        // Delta / inv arrived with the Q tile
      if (!(ok = g.wait(&sm.s_full, i & 1, 171))) break;
      tc_fence_after();
      // bias of query column c: -slope |key - (qi BLK + c)| = -sl * c + base with sl = slope for queries from the key on,
      // -slope for queries before it (non-causal only); MODE 1: causal diagonal tile (queries before the key are masked),
      // MODE 2: non-causal diagonal tile (absolute value element by element, nothing masked)
      const float sl = (!p.causal && qi < kt) ? -slope : slope;
      const float base = (!MASKED || kept) ? sl * float(key - qi * BLK) : kMaskedKeyBias;
      const f32x2 step2 = pk2(-2.f * sl, -2.f * sl);
      const float* iv = sm.inv[st];
      auto phase_a = [&](auto MODE, auto HL) { // the diagonal tile gets its own copy (no run-time test in the unrolled body)
        constexpr int kMode = decltype(MODE)::value;
        constexpr bool kHiLo = decltype(HL)::value && std::is_same<T, __nv_bfloat16>::value;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          uint32_t sreg[32], preg[16], lreg[kHiLo ? 16 : 1];
          tmem_ld32(tmem_addr(tS, lane_base, kColsPerGroup * w + 32 * c), sreg);
          tmem_wait_ld_regs(sreg);
          const int col0 = kColsPerGroup * w + 32 * c;
          f32x2 bias2 = pk2(fmaf(-sl, float(col0), base), fmaf(-sl, float(col0 + 1), base));
          float4 ivq = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            if (e % 2 == 0) ivq = *reinterpret_cast<const float4*>(iv + col0 + 2 * e);
            const f32x2 iv2 = e % 2 == 0 ? pk2(ivq.x, ivq.y) : pk2(ivq.z, ivq.w);
            f32x2 F2, g2, b2 = bias2;
            if constexpr (kMode == 2) {
              float b0, b1;
              upk2(bias2, b0, b1);
              b2 = pk2(-fabsf(b0), -fabsf(b1));
            }
            const f32x2 acc2 = pk2(__uint_as_float(sreg[2 * e]), __uint_as_float(sreg[2 * e + 1]));
            if (rcp_shared(e, FAT_RCP_SHARE_BWD)) score_fg2<true, true>(acc2, scale2, b2, one2, F2, g2);
            else                                  score_fg2<true, false>(acc2, scale2, b2, one2, F2, g2);
            bias2 = add2(bias2, step2);
            F2 = mul2(F2, iv2);
            g2 = mul2(g2, iv2);
            float p0, p1;
            upk2(F2, p0, p1);
            if constexpr (kMode == 1) {                       // queries before the key see nothing of it
              float g0, g1;
              upk2(g2, g0, g1);
              if (col0 + 2 * e < r) { p0 = 0.f; g0 = 0.f; }
              if (col0 + 2 * e + 1 < r) { p1 = 0.f; g1 = 0.f; }
              g2 = pk2(g0, g1);
            }
            gq[16 * c + e] = g2;
            preg[e] = Pack16<T>::pack(p0, p1);
            if constexpr (kHiLo) lreg[e] = pack_residual(p0, p1, preg[e]);
          }
          if constexpr (kHiLo) {
            tmem_st16(tmem_addr(tS, lane_base, col0), preg);
            tmem_st16(tmem_addr(tS, lane_base, col0 + 16), lreg);
          } else {
            tmem_st16(tmem_addr(tS, lane_base, packed_col(w, c)), preg);
          }
        }
      };
      if (!diag)         phase_a(std::integral_constant<int, 0>{}, std::integral_constant<bool, hilo>{});
      else if (p.causal) phase_a(std::integral_constant<int, 1>{}, std::integral_constant<bool, hilo>{});
      else               phase_a(std::integral_constant<int, 2>{}, std::integral_constant<bool, hilo>{});
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_full);
      // ---- phase B: dS^T = g (dP^T - Delta[q]) -> shared memory
      // dP^T(i) was committed by the issuer of dQ^T(i-1) and dK(i-1), after them: its barrier also says that those
      // have finished reading the dS^T tile
      if (!(ok = g.wait(&sm.dp_full, i & 1, 172))) break;
      tc_fence_after();
      const float* dl = sm.delta[st];
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        uint32_t dreg[32], preg[16];
        const int col0 = kColsPerGroup * w + 32 * c;
        tmem_ld32(tmem_addr(tP, lane_base, col0), dreg);
        tmem_wait_ld_regs(dreg);
        float4 dq4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (e % 2 == 0) dq4 = *reinterpret_cast<const float4*>(dl + col0 + 2 * e);
          const float2 d2 = e % 2 == 0 ? make_float2(dq4.x, dq4.y) : make_float2(dq4.z, dq4.w);
          const f32x2 ds2 = mul2(gq[16 * c + e], fma2(pk2(__uint_as_float(dreg[2 * e]), __uint_as_float(dreg[2 * e + 1])), cs2, pk2(-cs * d2.x, -cs * d2.y)));
          float d0, d1;
          upk2(ds2, d0, d1);
          preg[e] = pack_ds(d0, d1);
        }
#pragma unroll
        for (int sgm = 0; sgm < 4; ++sgm)        // 64-query chunk w of the tile, 16-byte segments 4c..4c+3 of this key's row
          *reinterpret_cast<uint4*>(sm.ds + w * (BLK * 128) + sw128_offset(r, 4 * c + sgm)) =
              make_uint4(preg[4 * sgm], preg[4 * sgm + 1], preg[4 * sgm + 2], preg[4 * sgm + 3]);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&sm.ds_full);
    }
    if (ok) ok = g.wait(&sm.acc_full, 0, 174);
    named_barrier(1, kEwThreads);
    if (!g.aborted()) {
      // d_v (staged in q[0]) and d_k (staged in dout[0]); the multipliers undo the 16x (F16) and 8x (g8) units
      tc_fence_after();
      for (int ch = w; ch < 2 * D / 32; ch += kEwGroups) {
        const bool is_dk = ch >= D / 32;
        const int c0 = (is_dk ? ch - D / 32 : ch) * 32;
        uint32_t oreg[32];
        tmem_ld32(tmem_addr(is_dk ? tK : tV, lane_base, c0), oreg);
        tmem_wait_ld_regs(oreg);
        stage_row32<T>(is_dk ? sm.dout : sm.q[0], r, c0, oreg, is_dk ? 0.25f * scale * dscale_inv / kDsScale : 0.0625f / kOpScale);
      }
      fence_async_smem();
      named_barrier(1, kEwThreads);
      if (tid == 0) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_store_4d(&maps.dv, sm.q[0] + c * (BLK * 128), c * 64, kt * BLK, h, b);
          tma_store_4d(&maps.dk, sm.dout + c * (BLK * 128), c * 64, kt * BLK, h, b);
        }
        tma_store_commit();
        tma_store_wait_all();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kFusedTmaWarp) tmem_dealloc(tmem, kTmemCols);
}

// d_q = round(dq_acc * scale / (4 kDsScale c)): float32 accumulator (dense [B,H,T,D]) -> tensor dtype with the caller's strides.
// One block = kConvRows rows of one (batch, head); a thread converts 8 values of kConvRows / (256 / (D/8)) rows.
constexpr int kConvRows = 64;
template <typename T, int D>
__global__ void __launch_bounds__(256)
attn_bwd_dq_convert_kernel(const AttnParams p, const float* __restrict__ dq_acc) {
  constexpr int PPR = D / 8, RPP = 256 / PPR;     // packs per row, rows per pass of the block
  const unsigned chunks = unsigned((p.T + kConvRows - 1) / kConvRows);
  const int bh = int(blockIdx.x / chunks), t0 = int(blockIdx.x % chunks) * kConvRows;
  const int b = bh / p.H, h = bh % p.H;
  const int c = int(threadIdx.x % PPR) * 8, tr = int(threadIdx.x / PPR);
  const float* src = dq_acc + int64_t(bh) * p.T * D + c;
  T* dst = static_cast<T*>(p.d_q) + b * p.dqs[0] + h * p.dqs[1] + c;
  float dscale, dscale_inv;
  dout_scale(dmax_of(p)[bh], dscale, dscale_inv);
  const float mul = 0.25f * p.scale * dscale_inv / kDsScale;     // undoes the g8 units and the operand scale of dS
#pragma unroll
  for (int i = 0; i < kConvRows / RPP; ++i) {
    const int t = t0 + tr + i * RPP;
    if (t < p.T) {
      const float4 lo = __ldcs(reinterpret_cast<const float4*>(src + int64_t(t) * D));
      const float4 hi = __ldcs(reinterpret_cast<const float4*>(src + int64_t(t) * D + 4));
      const float v[8] = {lo.x * mul, lo.y * mul, lo.z * mul, lo.w * mul, hi.x * mul, hi.y * mul, hi.z * mul, hi.w * mul};
      store_pack<T, 8>(dst + int64_t(t) * p.dqs[2], v);
    }
  }
}

size_t round1k(size_t n) { return (n + 1023) / 1024 * 1024; }
size_t stats_bytes(int B, int H, int T) { return round1k((2 * size_t(B) * H * pad_rows(T) + size_t(B) * H) * sizeof(float)); }
size_t dq_acc_bytes(int B, int H, int T, int D) { return round1k(size_t(B) * H * T * D * sizeof(float)); }
size_t f16_copy_bytes(int B, int H, int T, int D) { return round1k(size_t(B) * H * T * D * sizeof(__half)); }

// Workspace after the head described at dmax_of(): the float32 d_q accumulator of the fused kernel, then (bfloat16
// tensors only) the float16 copies of q and k, dense [B,H,T,D].
float* ws_dq_acc(const AttnParams& p) {
  return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p.delta) + stats_bytes(p.B, p.H, p.T));
}
__half* ws_q16(const AttnParams& p) {
  return reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(ws_dq_acc(p)) + dq_acc_bytes(p.B, p.H, p.T, p.D));
}
__half* ws_k16(const AttnParams& p) {
  return reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(ws_q16(p)) + f16_copy_bytes(p.B, p.H, p.T, p.D));
}

// dq_zero: the fused backward's float32 d_q accumulator, cleared by the same pass (nullptr: nothing to clear)
// copy_k: also write the float16 copy of k (the fused kernel converts its K tile itself and does not need it)
template <typename T, int D>
int launch_prepare(const AttnParams& p, cudaStream_t st, float* dq_zero, bool copy_k) {
  float* inv_rows = p.delta + int64_t(p.B) * p.H * pad_rows(p.T);
  const unsigned blocks = unsigned(p.B) * p.H * unsigned(pad_rows(p.T) / kPrepRows);
  if (cudaMemsetAsync(dmax_of(p), 0, size_t(p.B) * p.H * sizeof(uint32_t), st) != cudaSuccess) return check_launch("attn_bwd_prepare (clear)");
  constexpr bool kCopies = !std::is_same<T, __half>::value;
  attn_bwd_prepare_kernel<T, D><<<blocks, 256, 0, st>>>(p, inv_rows, dmax_of(p), dq_zero, kCopies ? ws_q16(p) : nullptr,
                                                        kCopies && copy_k ? ws_k16(p) : nullptr);
  return check_launch("attn_bwd_prepare");
}

// Tensor maps of the q and k operands of the main kernels: for bfloat16 tensors the float16 copies (dense), except
// that a kernel which converts its K tile itself (k_copy = false) reads k in place; for float16 the tensors themselves.
template <typename T, int D>
bool make_qk_maps(const AttnParams& p, CUtensorMap* mq, CUtensorMap* mk, bool k_copy) {
  const bool copies = !std::is_same<T, __half>::value;
  const int64_t dense[3] = {int64_t(p.H) * p.T * D, int64_t(p.T) * D, D};
  const bool ok_q = copies ? make_tmap_bhtd(mq, ws_q16(p), p.B, p.H, p.T, D, dense, 64, BLK)
                           : make_tmap_bhtd(mq, p.q, p.B, p.H, p.T, D, p.qs, 64, BLK);
  const bool ok_k = copies && k_copy ? make_tmap_bhtd(mk, ws_k16(p), p.B, p.H, p.T, D, dense, 64, BLK)
                                     : make_tmap_bhtd(mk, p.k, p.B, p.H, p.T, D, p.ks, 64, BLK);
  return ok_q && ok_k;
}

template <typename Kern, typename Maps>
int launch_main(Kern kern, const Maps& maps, const AttnParams& p, size_t smem, int threads, cudaStream_t st, const char* what) {
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    set_error("%s: cannot reserve %zu bytes of shared memory", what, smem);
    return FAT_ERR_LAUNCH;
  }
  const dim3 grid(banded_grid((p.T + BLK - 1) / BLK, p.B * p.H, kBwdBands));
  kern<<<grid, threads, smem, st>>>(maps, p);
  return check_launch(what);
}

// Deterministic backward: prepare, query-major d_q kernel, key-major d_k/d_v kernel.
template <typename T, int D>
int launch_bwd_split(const AttnParams& p, cudaStream_t st) {
  DqMaps mq;
  DkvMaps mk;
  if (!make_qk_maps<T, D>(p, &mq.q, &mq.k, true) ||
      !make_tmap_bhtd(&mq.dout, p.d_out, p.B, p.H, p.T, D, p.dos, 64, BLK) ||
      !make_tmap_bhtd(&mq.v, p.v, p.B, p.H, p.T, D, p.vs, 64, BLK) ||
      !make_tmap_bhtd(&mq.dq, p.d_q, p.B, p.H, p.T, D, p.dqs, 64, BLK) ||
      !make_tmap_bhtd(&mk.dk, p.d_k, p.B, p.H, p.T, D, p.dks, 64, BLK) ||
      !make_tmap_bhtd(&mk.dv, p.d_v, p.B, p.H, p.T, D, p.dvs, 64, BLK))
    return FAT_ERR_LAUNCH;
  mk.q = mq.q; mk.dout = mq.dout; mk.k = mq.k; mk.v = mq.v;
  if (int rc = launch_prepare<T, D>(p, st, nullptr, true)) return rc;
  if (int rc = launch_main(attn_bwd_dq_tc_kernel<T, D>, mq, p, sizeof(DqSmem<D>) + 1024, kBwdThreads, st, "attn_bwd_dq_tc")) return rc;
  if (p.key_mask) return launch_main(attn_bwd_dkv_tc_kernel<T, D, true>, mk, p, sizeof(DkvSmem<D>) + 1024, kBwdThreads, st, "attn_bwd_dkv_tc");
  return launch_main(attn_bwd_dkv_tc_kernel<T, D, false>, mk, p, sizeof(DkvSmem<D>) + 1024, kBwdThreads, st, "attn_bwd_dkv_tc");
}

// Fused backward: prepare (which also clears the float32 d_q accumulator), fused kernel, convert d_q.
template <typename T, int D>
int launch_bwd_fused(const AttnParams& p, cudaStream_t st) {
  float* dq_acc = ws_dq_acc(p);
  auto kern = p.key_mask ? attn_bwd_fused_tc_kernel<T, D, true> : attn_bwd_fused_tc_kernel<T, D, false>;
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
      fa.numRegs * kFusedThreads < 256 * kFusedRegsEw + 128 * kFusedRegsDrain + 128 * kFusedRegsAux) {
    // the warpgroups could never collect their register shares: refuse instead of letting setmaxnreg.inc wait
    set_error("attn_bwd_fused: built with %d registers per thread, the register hand-over needs %d", fa.numRegs, kFusedRegsLaunch);
    return FAT_ERR_LAUNCH;
  }
  FusedMaps m;
  if (!make_qk_maps<T, D>(p, &m.q, &m.k, false) ||
      !make_tmap_bhtd(&m.dout, p.d_out, p.B, p.H, p.T, D, p.dos, 64, BLK) ||
      !make_tmap_bhtd(&m.v, p.v, p.B, p.H, p.T, D, p.vs, 64, BLK) ||
      !make_tmap_bhtd(&m.dk, p.d_k, p.B, p.H, p.T, D, p.dks, 64, BLK) ||
      !make_tmap_bhtd(&m.dv, p.d_v, p.B, p.H, p.T, D, p.dvs, 64, BLK) ||
      !make_tmap_bhtd_f32(&m.dq_acc, dq_acc, p.B, p.H, p.T, D, D, 32))
    return FAT_ERR_LAUNCH;
  if (int rc = launch_prepare<T, D>(p, st, dq_acc, false)) return rc;
  if (int rc = launch_main(kern, m, p, sizeof(FusedSmem<D>), kFusedThreads, st, "attn_bwd_fused_tc")) return rc;
  const unsigned blocks = unsigned(p.B) * p.H * unsigned((p.T + kConvRows - 1) / kConvRows);
  attn_bwd_dq_convert_kernel<T, D><<<blocks, 256, 0, st>>>(p, dq_acc);
  return check_launch("attn_bwd_dq_convert");
}

template <typename T>
int launch_bwd(const AttnParams& p, cudaStream_t st) {
  if (p.D == 128) return p.deterministic ? launch_bwd_split<T, 128>(p, st) : launch_bwd_fused<T, 128>(p, st);
  return p.deterministic ? launch_bwd_split<T, 64>(p, st) : launch_bwd_fused<T, 64>(p, st);
}

}  // namespace

size_t attn_bwd_tc_workspace_bytes(int B, int H, int T, int D, int dtype) {
  // Delta, kOpScale/(L+eps) (rows padded to whole tiles) and max|dO|; the float32 d_q accumulator of the fused kernel;
  // for bfloat16 tensors the float16 copies of q and k
  return stats_bytes(B, H, T) + dq_acc_bytes(B, H, T, D) + (dtype == FAT_BF16 ? 2 * f16_copy_bytes(B, H, T, D) : 0);
}

int attn_bwd_tc(const AttnParams& p, int dtype, cudaStream_t st) {
  if (dtype == FAT_BF16) return launch_bwd<__nv_bfloat16>(p, st);
  if (dtype == FAT_F16) return launch_bwd<__half>(p, st);
  set_error("attn_bwd_tc: unsupported dtype tag %d", dtype);
  return FAT_ERR_DTYPE;
}

}  // namespace fat
