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

// ------------------------------------------------------------------ CTA work order of the causal kernels
// Per (batch, head) there are n_tiles CTAs whose cost falls with their rank (rank 0 sees the most tiles of the other
// side).  Blocks are dispatched in index order; with all ranks of one (batch, head) adjacent, the last (batch, head)
// starts its longest CTA when almost nothing else is left and the GPU idles behind it.  The 1-D grid can therefore be
// ordered in bands of ranks: band 0 holds the longest ranks of every (batch, head), the last band the shortest; inside
// a band the ranks of one (batch, head) stay adjacent so that CTAs running together still share its tiles in L2.
// More bands shorten the tail but spread each (batch, head) over more of the launch; measured at B*H = 128, S = 4096:
// two bands are best for the forward (-2 %), four and more lose to L2 misses, and the backward kernels are best
// with one band (all ranks of a (batch, head) adjacent, long ranks first).
#ifndef FAT_FWD_BANDS
#define FAT_FWD_BANDS 2
#define FAT_BWD_BANDS 1
#endif
constexpr int kFwdBands = FAT_FWD_BANDS, kBwdBands = FAT_BWD_BANDS;
__host__ __device__ inline int band_size(int n_tiles, int bands) { return (n_tiles + bands - 1) / bands; }
inline unsigned banded_grid(int n_tiles, int n_bh, int bands) {
  const int bs = band_size(n_tiles, bands);
  return unsigned((n_tiles + bs - 1) / bs) * unsigned(n_bh) * unsigned(bs);
}
// false: this block is padding (rank beyond n_tiles) and must return at once
__device__ __forceinline__ bool banded_tile(int n_tiles, int n_bh, int bands, int& rank, int& bh) {
  const unsigned bs = unsigned(band_size(n_tiles, bands)), per_band = unsigned(n_bh) * bs;
  const unsigned band = blockIdx.x / per_band, rem = blockIdx.x % per_band;
  bh = int(rem / bs);
  rank = int(band * bs + rem % bs);
  return rank < n_tiles;
}

// ------------------------------------------------------------------ GEMM issue helpers (one thread)
// Descriptors are built once per shared-memory buffer; inside the loops a K-step only adds a constant
// to the address field, so issuing a whole 128x128x128 GEMM costs a few dozen instructions.
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) { return smem_desc_sw128(smem_u32(tile), 16, 1024); }
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile) { return smem_desc_sw128(smem_u32(tile), BLK * 128, 1024); }

// acc[128 x 128] = A B^T over the head dimension; A and B are K-major [128][D] tiles.
template <int D>
__device__ __forceinline__ void issue_gemm_nt(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
#pragma unroll
  for (int s = 0; s < D / 16; ++s) {
    const uint32_t off = ((s / 4) * (BLK * 128) + (s % 4) * 32) >> 4;
    mma_ss(d_tmem, adesc + off, bdesc + off, idesc, s > 0);
  }
}

// acc[128 x N] (+)= A B with A in TMEM (128 x 128, packed 16-bit) and B an MN-major [128][N] tile.
// CW: the packed A is stored in pieces, one per element-wise warpgroup: elements [CW*w, CW*w+CW) occupy the
// CW/2 columns that start at column CW*w (CW = 128: one contiguous run of 64 columns).
template <int CW>
__device__ __forceinline__ void issue_gemm_tn(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int s = 0; s < BLK / 16; ++s) {
    const uint32_t acol = uint32_t(CW * ((16 * s) / CW) + ((16 * s) % CW) / 2);
    mma_ts(d_tmem, a_tmem + acol, bdesc + ((s * 2048) >> 4), idesc, accumulate || s > 0);
  }
}

// The same product with the packed A kept as a bfloat16 value plus its rounding residual (two 16-bit pieces, 16 more
// significand bits for eight more MMAs).  Layout: the 32 elements of score chunk j (elements [32 j, 32 j + 32)) occupy
// the chunk's own 32 columns, values in the first 16, residuals in the last 16, so that a thread can store both as soon
// as it has read that chunk.
__device__ __forceinline__ void issue_gemm_tn_hilo(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int s = 0; s < BLK / 16; ++s) {
    const uint32_t acol = uint32_t(32 * (s / 2) + 8 * (s % 2));
    mma_ts(d_tmem, a_tmem + acol, bdesc + ((s * 2048) >> 4), idesc, accumulate || s > 0);
    mma_ts(d_tmem, a_tmem + acol + 16, bdesc + ((s * 2048) >> 4), idesc, true);
  }
}

// ------------------------------------------------------------------ packed fp32 pairs (sm_100 FFMA2 / FMUL2 / FADD2)
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Every kRcpShare*-th pair of scores takes its two reciprocals from one special-function op (0: never).
#ifndef FAT_RCP_SHARE_FWD
#define FAT_RCP_SHARE_FWD 2
#define FAT_RCP_SHARE_BWD 8
#endif
__device__ __forceinline__ constexpr bool rcp_shared(int i, int every) { return every > 0 && i % every == 0; }

// Reciprocals of two numbers >= 1.  SHARED: from ONE special-function op, 1/a = b * (1/(a b)),
// 1/b = a * (1/(a b)) (three extra multiplies); otherwise two special-function ops.  The kernels
// mix both so that neither the special-function pipe nor the FMA pipe becomes the limiter.
template <bool SHARED>
__device__ __forceinline__ f32x2 rcp_pair(float a, float b) {
  if (SHARED) {
    const float rr = rcp_approx(a * b);
    return pk2(b * rr, a * rr);
  }
  return pk2(rcp_approx(a), rcp_approx(b));
}

// For a packed pair of scores s: r = 1/(|s|+1) and w = 1 + s r = 2 sigma(s).
template <bool SHARED>
__device__ __forceinline__ void sigma_terms2(f32x2 s2, f32x2 one2, f32x2& r2, f32x2& w2) {
  float s0, s1;
  upk2(s2, s0, s1);
  r2 = rcp_pair<SHARED>(fabsf(s0) + 1.0f, fabsf(s1) + 1.0f);
  w2 = fma2(s2, r2, one2);
}

// Waits for this thread's outstanding TMEM loads.  The registers are listed as read-write operands so that
// the compiler cannot move arithmetic on them above the wait.
__device__ __forceinline__ void tmem_wait_ld_regs(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}

}  // namespace tcattn
}  // namespace fat
