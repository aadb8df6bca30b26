// Causal rational attention forward on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// One CTA owns 256 consecutive queries of one (batch, head): two 128-row query tiles, each
// served by kSplit "softmax" warpgroups (one thread per query row and share of the score columns).  A producer warp streams
// 128-key K and V tiles through a two-stage shared-memory ring with TMA; an issuer warp
// drives the tensor core:   S_t = Q_t K^T  (smem x smem -> TMEM, fp32)
//                           O_t += P_t V   (TMEM x smem -> TMEM, fp32)
// Because sigma(s)^4 lies in [0,1] there is no running maximum and nothing to rescale: the
// output accumulates in TMEM across all key tiles untouched by the CUDA cores, which only
// turn S into P = sigma(S*scale + alibi)^4 in place (16-bit, packed over the fp32 scores)
// and keep a running row sum.  The two query tiles ping-pong, so the tensor core works on
// one while the other is in its element-wise phase.
//
// P is always float16 (stored as 4096 sigma^4 <= 4096).  Rounded to bfloat16 its error moves the output
// by ~1e-3 |v| on rows that attend to a few keys: inside the output's own tolerance, but the backward
// forms Delta = dO . O from this output, where the error is amplified by sqrt(D) |dO| and puts a few
// elements in 10^4 of d_q outside the bar.  tcgen05.mma wants both operands of one MMA in one 16-bit
// format, so for bfloat16 tensors two helper warps turn every V tile into float16 in shared memory
// before O += P V reads it (exact for magnitudes in [2^-14, 65504], absolute error <= 2^-25 below;
// 65536 and more are clamped to 65504 and reported in bit 29 of the status word).  S = Q K^T uses
// q and k as they are.
//
// TMEM columns: S0/P0 [0,128)  S1/P1 [128,256)  O0 [256,256+D)  O1 [256+D,256+2D).
#include <type_traits>

#include "attn_tc_common.cuh"

namespace fat {
namespace {

using namespace tc;
using namespace tcattn;

constexpr int kStages = 2;                            // K tiles in flight
#ifndef FAT_FWD_VSTAGES
#define FAT_FWD_VSTAGES 3
#endif
constexpr int kVStages = FAT_FWD_VSTAGES;             // V tiles in flight (a V tile is loaded, converted, then read by two MMAs)
#ifndef FAT_FWD_CVT_WARPS
#define FAT_FWD_CVT_WARPS 2
#endif
#ifndef FAT_FWD_SPLIT
#define FAT_FWD_SPLIT 1
#endif
constexpr int kSplit = FAT_FWD_SPLIT;                 // softmax warpgroups per query tile (each takes 128/kSplit score columns)
constexpr int kEwWarps = 8 * kSplit;                  // softmax warps; then one TMA warp, one MMA warp and two helper warps
constexpr int kCvtWarps = FAT_FWD_CVT_WARPS;
constexpr int kFwdThreads = 32 * kEwWarps + 64 + 32 * kCvtWarps;
constexpr float kPUnit = 4096.0f;                     // P_stored = kPUnit sigma^4 = (4 (1 + s r))^4
constexpr int kStatusF16Range = 0x20000000;
constexpr int kColsPerWg = BLK / kSplit;
constexpr int kChunks = kColsPerWg / 32;

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = BLK * D * 2;          // one [128][D] 16-bit tile
  alignas(1024) unsigned char q[2][kTileBytes];           // reused as output staging in the epilogue
  alignas(1024) unsigned char k[kStages][kTileBytes];
  alignas(1024) unsigned char v[kVStages][kTileBytes];
  uint64_t q_full[2], k_full[kStages], k_empty[kStages], v_full[kVStages], v_empty[kVStages];
  uint64_t v_ready[kVStages];                              // helper warps: the V tile of this stage is float16 now
  uint64_t s_full[2], p_full[2], o_full[2];
  float l_part[2][kSplit][BLK];                           // row sums of each warpgroup's column share
  uint32_t tmem_base;
  int abort_flag;
};

struct FwdMaps { CUtensorMap q, k, v, out, out_lo; };

// One 32-column chunk of a thread's score row: S (fp32, registers sreg) -> P = (8 sigma(S*scale + bias))^4 = 4096 sigma^4
// as packed float16 pairs in preg (the factor cancels in O = P V / sum P); adds the chunk's row sum to l2.
// With r' = 1/((|s|+1)/4) = 4 r (one fused multiply-add feeds the reciprocal, as the plain |s|+1 would) and
// w' = 4 + s r' = 4 (1 + s r) = 8 sigma, the scaling costs no instruction.  `four2` holds the packed constant 4.
// The ALiBi bias of column c is slope * c + base (the caller gives slope and base the sign that makes it -slope_h |i - j|
// on its side of the diagonal).  MASK: keys with column index > lim get no weight (causal: the diagonal tile, lim = the
// thread's row; non-causal: the last key tile of a ragged sequence, lim = its last valid column).  ABS: the tile
// straddles the diagonal of a non-causal problem, the bias is -|slope * c + base|.
template <bool MASK, bool ABS, bool KM>
__device__ __forceinline__ void softmax_chunk(const uint32_t (&sreg)[32], uint32_t (&preg)[16], int c, int lim, uint32_t keep,
                                              f32x2 scale2, f32x2 four2, f32x2 step2, float slope, float base, f32x2& l2) {
  f32x2 bias2 = pk2(fmaf(slope, float(c * 32), base), fmaf(slope, float(c * 32 + 1), base));
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    f32x2 b2 = bias2;
    if (ABS) {
      float b0, b1;
      upk2(bias2, b0, b1);
      b2 = pk2(-fabsf(b0), -fabsf(b1));
    }
    const f32x2 s2 = fma2(pk2(__uint_as_float(sreg[2 * i]), __uint_as_float(sreg[2 * i + 1])), scale2, b2);
    bias2 = add2(bias2, step2);
    float s0, s1;
    upk2(s2, s0, s1);
    const float a0 = fmaf(fabsf(s0), 0.25f, 0.25f), a1 = fmaf(fabsf(s1), 0.25f, 0.25f);
    const f32x2 r2 = rcp_shared(i, FAT_RCP_SHARE_FWD) ? rcp_pair<true>(a0, a1) : rcp_pair<false>(a0, a1);
    const f32x2 w2 = fma2(s2, r2, four2);
    const f32x2 q2 = mul2(w2, w2);
    f32x2 f2 = mul2(q2, q2);                               // (8 sigma)^4 = 4096 sigma^4
    float f0, f1;
    upk2(f2, f0, f1);
    if (KM) {                                              // `keep` already holds the limit, if there is one
      if (!(keep & (1u << (2 * i)))) f0 = 0.f;
      if (!(keep & (2u << (2 * i)))) f1 = 0.f;
      f2 = pk2(f0, f1);
    } else if (MASK) {
      if (c * 32 + 2 * i > lim) f0 = 0.f;
      if (c * 32 + 2 * i + 1 > lim) f1 = 0.f;
      f2 = pk2(f0, f1);
    }
    l2 = add2(l2, f2);
    preg[i] = Pack16<__half>::pack(f0, f1);
  }
}

// A thread's share of one score row: kChunks 32-column chunks starting at TMEM address `trow` (absolute chunk
// index c0).  The packed P of chunk c lands on columns [16 c, 16 c + 16) counted from `trow`, i.e. over scores
// this thread has already taken into registers.  The chunk loop is kept rolled (the body is ~400 instructions;
// unrolled four times it no longer fits the instruction cache).
// KM: a padding mask over the keys is in force; `keep_words` points at the four 32-bit words of this key tile (bit set =
// the key takes part) and MASK's limit, if any, is folded into the word of each chunk.
template <bool MASK, bool ABS, bool KM = false>
__device__ __forceinline__ void softmax_tile(uint32_t trow, int c0, int lim, f32x2 scale2, f32x2 four2, f32x2 step2,
                                             float slope, float base, f32x2& l2, const uint32_t* keep_words = nullptr) {
  uint32_t sreg[32];
  tmem_ld32(trow, sreg);
#pragma unroll 1
  for (int c = 0; c < kChunks; ++c) {
    uint32_t keep = 0xffffffffu;
    if (KM) {
      keep = __ldg(keep_words + c0 + c);
      if (MASK) {
        const int rel = lim - (c0 + c) * 32;                 // last column of this chunk that may be seen
        keep &= rel >= 31 ? 0xffffffffu : (rel < 0 ? 0u : (2u << rel) - 1u);
      }
    }
    tmem_wait_ld_regs(sreg);
    uint32_t preg[16];
    softmax_chunk<MASK, ABS, KM>(sreg, preg, c0 + c, lim, keep, scale2, four2, step2, slope, base, l2);
    if (c + 1 < kChunks) tmem_ld32(trow + (c + 1) * 32, sreg);      // next chunk in flight while this one is stored
    tmem_st16(trow + c * 16, preg);
  }
}

// bfloat16 -> float16 in place over `BYTES` bytes of a shared-memory tile, by the 32 lanes of one warp.  CHECK: returns
// non-zero when a magnitude was 65536 or more (or not a number); such values are clamped to 65504.
template <int BYTES, bool CHECK>
__device__ __forceinline__ uint32_t convert_v(unsigned char* base, int lane) {
  uint32_t flag = 0;
#pragma unroll 4
  for (int off = lane * 16; off < BYTES; off += 32 * 16) {
    uint4 v = *reinterpret_cast<uint4*>(base + off);
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t x = w[i];
      if (CHECK) flag |= ((x & 0x7fff7fffu) + 0x38803880u) & 0x80008000u;          // either half >= 0x4780 (65536.0)
      uint32_t y;
      asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(__uint_as_float(x & 0xffff0000u)), "f"(__uint_as_float(x << 16)));
      w[i] = y;
    }
    *reinterpret_cast<uint4*>(base + off) = v;
  }
  return flag;
}

template <typename T, int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_tc_kernel(const __grid_constant__ FwdMaps maps, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  using S = FwdSmem<D>;
  S& sm = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_qb = (p.T + 2 * BLK - 1) / (2 * BLK);
  int rank, bh;
  if (!banded_tile(n_qb, p.B * p.H, kFwdBands, rank, bh)) return;      // padding block of the banded order
  const int b = bh / p.H, h = bh % p.H;
  const int qb = n_qb - 1 - rank;                            // long query blocks first
  const int n_kv_total = (p.T + BLK - 1) / BLK;
  // query tile t covers rows [(2qb+t)*128, +128); it needs key tiles 0..(2qb+t) (causal)
  int n_tiles[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) n_tiles[t] = (2 * qb + t) * BLK < p.T ? (p.causal ? min(2 * qb + t + 1, n_kv_total) : n_kv_total) : 0;
  const int n_max = max(n_tiles[0], n_tiles[1]);
  Guard g{&sm.abort_flag, p.status};
  constexpr bool kConvertV = !std::is_same<T, __half>::value;

  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1); mbar_init(&sm.s_full[i], 1); mbar_init(&sm.p_full[i], BLK * kSplit); mbar_init(&sm.o_full[i], 1);
    }
    for (int i = 0; i < kStages; ++i) { mbar_init(&sm.k_full[i], 1); mbar_init(&sm.k_empty[i], 1); }
    for (int i = 0; i < kVStages; ++i) {
      mbar_init(&sm.v_full[i], 1); mbar_init(&sm.v_empty[i], 1); mbar_init(&sm.v_ready[i], 32 * kCvtWarps);
    }
    mbar_fence_init();
  }
  if (warp == kEwWarps) { tmem_alloc(&sm.tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == kEwWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&maps.q); tma_prefetch_desc(&maps.k); tma_prefetch_desc(&maps.v);
      for (int t = 0; t < 2; ++t)
        if (n_tiles[t] > 0) load_tile_tma<D>(sm.q[t], &maps.q, &sm.q_full[t], (2 * qb + t) * BLK, h, b);
      for (int j = 0; j < n_max; ++j) {
        const int st = j % kStages, vst = j % kVStages;
        if (!g.wait(&sm.k_empty[st], ((j / kStages) & 1) ^ 1, 10)) break;
        load_tile_tma<D>(sm.k[st], &maps.k, &sm.k_full[st], j * BLK, h, b);
        if (!g.wait(&sm.v_empty[vst], ((j / kVStages) & 1) ^ 1, 11)) break;
#ifdef FAT_TEST_WITHHOLD_V_TILE
        // test builds only (never the shipped library): this V tile is not loaded, so every wait that depends on it
        // runs out, which is how the give-up path (status word, teardown, TMEM release) gets exercised
        if (j == FAT_TEST_WITHHOLD_V_TILE) continue;
#endif
        load_tile_tma<D>(sm.v[vst], &maps.v, &sm.v_full[vst], j * BLK, h, b);
      }
    }
  } else if (warp == kEwWarps + 1) {
    // ------------------------------------------------------------------ tensor-core issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = idesc_f16(BLK, BLK, Pack16<T>::kFmt, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(BLK, D, Pack16<__half>::kFmt, 0, 1);      // P and V are float16
      const uint64_t qd[2] = {desc_kmajor(sm.q[0]), desc_kmajor(sm.q[1])};
      const uint64_t kd[kStages] = {desc_kmajor(sm.k[0]), desc_kmajor(sm.k[1])};
      uint64_t vd[kVStages];
#pragma unroll
      for (int i = 0; i < kVStages; ++i) vd[i] = desc_mnmajor(sm.v[i]);
      auto issue_qk = [&](int t, int st) { issue_gemm_nt<D>(tmem + t * BLK, qd[t], kd[st], idesc_qk); };          // S_t = Q_t K^T
      auto issue_pv = [&](int t, int st, bool first) {                                                           // O_t += P_t V
        issue_gemm_tn<kColsPerWg>(tmem + 2 * BLK + t * D, tmem + t * BLK, vd[st], idesc_pv, !first);
      };
      bool ok = true;
      // prologue: scores of key tile 0 for both query tiles
      if (n_max > 0) ok = g.wait(&sm.k_full[0], 0, 20);
      for (int t = 0; t < 2 && ok; ++t) {
        if (n_tiles[t] == 0) continue;
        ok = g.wait(&sm.q_full[t], 0, 21);
        if (!ok) break;
        tc_fence_after();
        issue_qk(t, 0);
        mma_commit(&sm.s_full[t]);
      }
      if (ok && n_max > 0) mma_commit(&sm.k_empty[0]);
      for (int j = 0; j < n_max && ok; ++j) {
        const int st1 = (j + 1) % kStages, vst = j % kVStages;
        const uint32_t ph1 = ((j + 1) / kStages) & 1, vph = (j / kVStages) & 1;
        bool k_next_ready = false;
        // V(j) and K(j+1) were requested an iteration or more ago: their barriers are settled first, so that nothing but the
        // issue of the MMAs stands between a tile's P and its next S (a satisfied wait still costs 150-250 cycles)
        if (!(ok = g.wait_polling(kConvertV ? &sm.v_ready[vst] : &sm.v_full[vst], vph, 23))) break;
        if (j + 1 < n_max) { if (!(ok = g.wait_polling(&sm.k_full[st1], ph1, 24))) break; k_next_ready = true; }
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= n_tiles[t]) continue;
          if (!(ok = g.wait_polling(&sm.p_full[t], j & 1, 22))) break;
          tc_fence_after();
          issue_pv(t, vst, j == 0);
          if (j + 1 < n_tiles[t]) {
            issue_qk(t, st1);
            mma_commit(&sm.s_full[t]);
          } else {
            mma_commit(&sm.o_full[t]);
          }
        }
        (void)k_next_ready;
        if (!ok) break;
        mma_commit(&sm.v_empty[vst]);                      // V(j) and, if it was read, K(j+1) are free once these finish
        if (j + 1 < n_max) mma_commit(&sm.k_empty[st1]);
      }
    }
  } else if (warp >= kEwWarps + 2) {
    // ------------------------------------------------------------------ helper warps: V tiles bfloat16 -> float16 in place
    // (every element keeps its place, so the swizzle does not matter).  Each V tile belongs to the CTA whose
    // query block starts at it; that CTA checks its range.
    if (kConvertV) {
      const int part = warp - (kEwWarps + 2), lane = tid & 31;
      constexpr int kPartBytes = S::kTileBytes / kCvtWarps;
      uint32_t out_of_range = 0;
      for (int j = 0; j < n_max; ++j) {
        const int st = j % kVStages;
        if (!g.wait(&sm.v_full[st], (j / kVStages) & 1, 40)) break;
        unsigned char* base = sm.v[st] + part * kPartBytes;
        if (j / 2 == qb) out_of_range |= convert_v<kPartBytes, true>(base, lane);
        else             convert_v<kPartBytes, false>(base, lane);
        fence_async_smem();
        mbar_arrive(&sm.v_ready[st]);
      }
      if (out_of_range && p.status) atomicOr(p.status, kStatusF16Range);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int t = (warp >> 2) / kSplit;                      // query tile of this warpgroup
    const int part = (warp >> 2) % kSplit;                   // which share of the score columns
    const int r = tid & (BLK - 1);                           // row inside the tile == TMEM lane
    const int row = (2 * qb + t) * BLK + r;                  // query index
    const uint32_t lane_base = uint32_t(warp & 3) * 32;
    const float slope = p.slopes[h];
    const float scale = p.scale;
    const int n = n_tiles[t];
    f32x2 l2 = pk2(0.f, 0.f);
    const f32x2 scale2 = pk2(scale, scale), four2 = pk2(4.0f, 4.0f);
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (!(ok = g.wait(&sm.s_full[t], j & 1, 30))) break;
      tc_fence_after();
      const bool diag = (j == 2 * qb + t);
      // bias of column c of this tile: -slope |row - (j BLK + c)|.  Keys up to the query: slope * c + slope (j BLK - row);
      // keys after it (non-causal only): the same with the sign flipped; the diagonal tile of a non-causal problem
      // takes the absolute value element by element.
      const float sl = (!p.causal && j > 2 * qb + t) ? -slope : slope;
      const float base = sl * float(j * BLK - row);
      const f32x2 step2 = pk2(2.f * sl, 2.f * sl);
      const uint32_t trow = tmem_addr(tmem, lane_base, t * BLK + part * kColsPerWg);
      if (p.key_mask) {
        // (bits of keys beyond T are clear, so a ragged last tile needs no limit of its own)
        const uint32_t* kw = p.key_mask + int64_t(b) * p.mask_words + j * (BLK / 32);
        if (p.causal && diag) softmax_tile<true, false, true>(trow, part * kChunks, r, scale2, four2, step2, sl, base, l2, kw);
        else if (diag)        softmax_tile<false, true, true>(trow, part * kChunks, 0, scale2, four2, step2, sl, base, l2, kw);
        else                  softmax_tile<false, false, true>(trow, part * kChunks, 0, scale2, four2, step2, sl, base, l2, kw);
      } else if (p.causal) {
        if (diag) softmax_tile<true, false>(trow, part * kChunks, r, scale2, four2, step2, sl, base, l2);
        else      softmax_tile<false, false>(trow, part * kChunks, r, scale2, four2, step2, sl, base, l2);
      } else {
        // zero-filled keys beyond T are not neutral (sigma(bias)^4 > 0): the last tile of a ragged sequence masks them
        const int last_col = p.T - 1 - j * BLK;
        const bool tail = last_col < BLK - 1;
        if (diag && tail)  softmax_tile<true, true>(trow, part * kChunks, last_col, scale2, four2, step2, sl, base, l2);
        else if (diag)     softmax_tile<false, true>(trow, part * kChunks, 0, scale2, four2, step2, sl, base, l2);
        else if (tail)     softmax_tile<true, false>(trow, part * kChunks, last_col, scale2, four2, step2, sl, base, l2);
        else               softmax_tile<false, false>(trow, part * kChunks, 0, scale2, four2, step2, sl, base, l2);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm.p_full[t]);
    }
    float l_sum;
    {
      float la, lb;
      upk2(l2, la, lb);
      l_sum = (la + lb) * (1.0f / kPUnit);                     // back to sum of sigma^4
    }
    if (kSplit > 1) sm.l_part[t][part][r] = l_sum;
    if (ok && n > 0) ok = g.wait(&sm.o_full[t], 0, 31);
    named_barrier(1 + t, BLK * kSplit);                      // reached by all of the tile's threads, aborted or not
    if (kSplit > 1) {
      l_sum = 0.f;
#pragma unroll
      for (int i = 0; i < kSplit; ++i) l_sum += sm.l_part[t][i][r];
    }
    if (n > 0 && !g.aborted()) {
      // -------------------------------------------------------------- epilogue: O / (L + eps), hi + residual
      tc_fence_after();
      const float inv = (1.0f / kPUnit) / (l_sum + p.eps);     // the accumulator holds kPUnit sigma^4 V
      if (part == 0 && row < p.T) p.L[(int64_t(b) * p.H + h) * p.T + row] = l_sum;
      unsigned char* stage = sm.q[t];
      const bool want_lo = p.out_lo != nullptr;
      for (int pass = 0; pass < (want_lo ? 2 : 1); ++pass) {
#pragma unroll
        for (int cc = 0; cc < D / 32 / kSplit; ++cc) {
          const int c = part * (D / 32 / kSplit) + cc;       // each warpgroup converts its share of the D columns
          uint32_t oreg[32];
          tmem_ld32(tmem_addr(tmem, lane_base, 2 * BLK + t * D + c * 32), oreg);
          tmem_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = __uint_as_float(oreg[2 * i]) * inv, bb = __uint_as_float(oreg[2 * i + 1]) * inv;
            uint32_t hi = Pack16<T>::pack(a, bb);
            if (pass == 1) { const float2 hf = Pack16<T>::unpack(hi); hi = Pack16<T>::pack(a - hf.x, bb - hf.y); }
            w[i] = hi;
          }
#pragma unroll
          for (int sgm = 0; sgm < 4; ++sgm) {
            const int col = c * 32 + sgm * 8;                 // first column of this 16-byte segment
            *reinterpret_cast<uint4*>(stage + (col / 64) * (BLK * 128) + sw128_offset(r, (col % 64) / 8)) =
                make_uint4(w[4 * sgm], w[4 * sgm + 1], w[4 * sgm + 2], w[4 * sgm + 3]);
          }
        }
        fence_async_smem();
        named_barrier(1 + t, BLK * kSplit);
        if (r == 0 && part == 0) {
          const CUtensorMap* m = pass == 0 ? &maps.out : &maps.out_lo;
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_store_4d(m, stage + c * (BLK * 128), c * 64, (2 * qb + t) * BLK, h, b);
          tma_store_commit();
          tma_store_wait_read();
        }
        named_barrier(1 + t, BLK * kSplit);
      }
      if (r == 0 && part == 0) tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kEwWarps) tmem_dealloc(tmem, kTmemCols);
}

template <typename T, int D>
int launch_fwd(const AttnParams& p, cudaStream_t st) {
  FwdMaps maps;
  if (!make_tmap_bhtd(&maps.q, p.q, p.B, p.H, p.T, D, p.qs, 64, BLK) ||
      !make_tmap_bhtd(&maps.k, p.k, p.B, p.H, p.T, D, p.ks, 64, BLK) ||
      !make_tmap_bhtd(&maps.v, p.v, p.B, p.H, p.T, D, p.vs, 64, BLK) ||
      !make_tmap_bhtd(&maps.out, p.out, p.B, p.H, p.T, D, p.os, 64, BLK))
    return FAT_ERR_LAUNCH;
  if (p.out_lo) {
    if (!make_tmap_bhtd(&maps.out_lo, p.out_lo, p.B, p.H, p.T, D, p.os, 64, BLK)) return FAT_ERR_LAUNCH;
  } else {
    maps.out_lo = maps.out;
  }
  auto kern = attn_fwd_tc_kernel<T, D>;
  const size_t smem = sizeof(FwdSmem<D>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) { set_error("attn_fwd_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return FAT_ERR_LAUNCH; }
  const dim3 grid(banded_grid((p.T + 2 * BLK - 1) / (2 * BLK), p.B * p.H, kFwdBands));
  kern<<<grid, kFwdThreads, smem, st>>>(maps, p);
  return check_launch("attn_fwd_tc");
}

}  // namespace

int attn_fwd_tc(const AttnParams& p, int dtype, cudaStream_t st) {
  if (dtype == FAT_BF16) return p.D == 128 ? launch_fwd<__nv_bfloat16, 128>(p, st) : launch_fwd<__nv_bfloat16, 64>(p, st);
  if (dtype == FAT_F16) return p.D == 128 ? launch_fwd<__half, 128>(p, st) : launch_fwd<__half, 64>(p, st);
  set_error("attn_fwd_tc: unsupported dtype tag %d", dtype);
  return FAT_ERR_DTYPE;
}

}  // namespace fat
