// Shifted cross-entropy of the language-model head in one pass over the logits.
//
// The reference computes  F.cross_entropy(logits[..., :-1, :].contiguous().view(-1, V), labels[..., 1:].view(-1),
// ignore_index=-100)  (algebraic_model.py:229-235): a copy of the logits, a log-softmax pass that writes a tensor of the
// same size, and in the backward a log-softmax-backward pass and a zero-padded slice gradient.  Here one kernel reads
// every logits row once and writes the row's loss and the row of d(loss)/d(logits) (already divided by the number of
// valid targets; zero for the last position of a sequence and for ignored targets).  Two kernels: 16-bit rows that fit
// shared memory at least twice go through persistent CTAs that stage whole rows with bulk asynchronous copies
// (shifted_ce_staged_kernel); everything else keeps the row in registers, one block per row (shifted_ce_kernel).  The
// backward only multiplies by the incoming scalar gradient, and skips even that when the scalar is 1.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "../../include/fat_b200.h"
#include "common.cuh"
#include "tc_common.cuh"

namespace fat {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kCePacks = 16;                       // 16-byte packs of one row a thread keeps in registers
#ifndef FAT_CE_STAGED
#define FAT_CE_STAGED 1
#endif
#ifndef FAT_CE_STAGED_THREADS
#define FAT_CE_STAGED_THREADS 512
#endif
constexpr int kCeStagedThreads = FAT_CE_STAGED_THREADS;
constexpr size_t kCeSmemBytes = 200 * 1024;        // shared memory the staged kernel may ask for

__device__ __forceinline__ float fast_exp2(float x) {      // x <= 0 here: flushing tiny results to zero is harmless
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NT>
__device__ __forceinline__ float block_reduce(float v, float* buf, bool is_max) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, m);
    v = is_max ? fmaxf(v, o) : v + o;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                                 // the previous use of buf has been read by everyone
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  float r = buf[0];
#pragma unroll
  for (int w = 1; w < NT / 32; ++w) r = is_max ? fmaxf(r, buf[w]) : r + buf[w];
  return r;
}

// One block of NT threads per row.  CACHED: the row is aligned and fits in kCePacks packs per thread; otherwise it is
// re-read from global memory (L2) for each of the three sweeps.  Rows of up to NT * kCePacks packs take the smaller
// block size, so that two or three blocks share an SM and fill each other's reduction barriers.
template <typename T, int kCeThreads, bool CACHED>
__global__ void __launch_bounds__(kCeThreads)
shifted_ce_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ n_valid,
                  float* __restrict__ row_loss, T* __restrict__ d_logits, int B, int Tn, int V,
                  int64_t ls_b, int64_t ls_t, int64_t lab_b, int64_t lab_t, int64_t ignore_index) {
  constexpr int W = 16 / sizeof(T);
  __shared__ float buf[kCeThreads / 32];
  const int tid = threadIdx.x;
  const float scale = 1.0f / fmaxf(n_valid[0], 1.0f);
  const int n_rows = B * Tn, npk = V / W;
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const int b = row / Tn, t = row - b * Tn;
    const T* x = logits + b * ls_b + t * ls_t;
    T* dx = d_logits ? d_logits + int64_t(row) * V : nullptr;     // null: the caller wants the loss only
    const int64_t target = t + 1 < Tn ? labels[b * lab_b + (t + 1) * lab_t] : ignore_index;
    const bool valid = target != ignore_index && target >= 0 && target < V;
    if (!valid) {                                  // uniform over the block
      if (!dx) {
      } else if (CACHED) {
        for (int pk = tid; pk < npk; pk += kCeThreads) reinterpret_cast<uint4*>(dx)[pk] = make_uint4(0u, 0u, 0u, 0u);
      } else {
        for (int c = tid; c < V; c += kCeThreads) dx[c] = Elem<T>::from_c(0.f);
      }
      if (tid == 0) row_loss[row] = 0.f;
      continue;
    }
    // d_logits may be the logits buffer itself (every element is read before the same thread overwrites it), so the
    // target's logit is fetched before anything is written
    const float x_target = tid == 0 ? Elem<T>::to_c(x[int(target)]) : 0.f;
    uint4 raw[kCePacks];
    float m = -INFINITY;
    if (CACHED) {
#pragma unroll
      for (int i = 0; i < kCePacks; ++i) {
        const int pk = tid + i * kCeThreads;
        if (pk < npk) {
          raw[i] = __ldcs(reinterpret_cast<const uint4*>(x) + pk);
          const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
          for (int j = 0; j < W; ++j) m = fmaxf(m, Elem<T>::to_c(e[j]));
        }
      }
    } else {
      for (int c = tid; c < V; c += kCeThreads) m = fmaxf(m, Elem<T>::to_c(x[c]));
    }
    m = block_reduce<kCeThreads>(m, buf, true);
    const float off = m * kLog2e;
    float s = 0.f;
    if (CACHED) {
#pragma unroll
      for (int i = 0; i < kCePacks; ++i) {
        if (tid + i * kCeThreads < npk) {
          const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
          for (int j = 0; j < W; ++j) s += fast_exp2(fmaf(Elem<T>::to_c(e[j]), kLog2e, -off));
        }
      }
    } else {
      for (int c = tid; c < V; c += kCeThreads) s += fast_exp2(fmaf(Elem<T>::to_c(x[c]), kLog2e, -off));
    }
    s = block_reduce<kCeThreads>(s, buf, false);
    const float inv = scale / s;                   // softmax normaliser and 1/n_valid in one factor
    const int tgt = int(target);
    if (!dx) {
    } else if (CACHED) {
#pragma unroll
      for (int i = 0; i < kCePacks; ++i) {
        const int pk = tid + i * kCeThreads;
        if (pk < npk) {
          const T* e = reinterpret_cast<const T*>(&raw[i]);
          float o[W];
#pragma unroll
          for (int j = 0; j < W; ++j) {
            o[j] = fast_exp2(fmaf(Elem<T>::to_c(e[j]), kLog2e, -off)) * inv;
            if (pk * W + j == tgt) o[j] -= scale;
          }
          store_pack<T, W>(dx + int64_t(pk) * W, o);
        }
      }
    } else {
      for (int c = tid; c < V; c += kCeThreads) {
        float o = fast_exp2(fmaf(Elem<T>::to_c(x[c]), kLog2e, -off)) * inv;
        if (c == tgt) o -= scale;
        dx[c] = Elem<T>::from_c(o);
      }
    }
    if (tid == 0) row_loss[row] = m + logf(s) - x_target;
  }
}

// Two neighbouring float32 values as one 64-bit register pair (fma.rn.f32x2 and mul.rn.f32x2 work on both at once), and a
// 16-byte pack of the tensor dtype as such pairs.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void upk2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

template <typename T> struct Pairs;
template <> struct Pairs<__nv_bfloat16> {
  static __device__ __forceinline__ void get(const uint4& raw, f32x2 (&o)[4]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = pk2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  static __device__ __forceinline__ void store(uint4* dst, const uint32_t (&w)[4]) { *dst = make_uint4(w[0], w[1], w[2], w[3]); }
  static __device__ __forceinline__ void stream(__nv_bfloat16* dst, const uint32_t (&w)[4]) { __stcs(reinterpret_cast<uint4*>(dst), make_uint4(w[0], w[1], w[2], w[3])); }
};
template <> struct Pairs<__half> {
  static __device__ __forceinline__ void get(const uint4& raw, f32x2 (&o)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); o[i] = pk2(f.x, f.y); }
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  static __device__ __forceinline__ void store(uint4* dst, const uint32_t (&w)[4]) { *dst = make_uint4(w[0], w[1], w[2], w[3]); }
  static __device__ __forceinline__ void stream(__half* dst, const uint32_t (&w)[4]) { __stcs(reinterpret_cast<uint4*>(dst), make_uint4(w[0], w[1], w[2], w[3])); }
};
// Largest element of the packs tid, tid + nt, ... of a 16-bit row in shared memory, compared two elements at a time
// without unpacking them.
template <typename T> struct RowMax;
template <> struct RowMax<__nv_bfloat16> {
  static __device__ __forceinline__ float of(const uint4* row, int tid, int npk, int nt) {
    __nv_bfloat162 m2 = __float2bfloat162_rn(-INFINITY);
#pragma unroll 4
    for (int pk = tid; pk < npk; pk += nt) {
      const uint4 raw = row[pk];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      m2 = __hmax2(__hmax2(m2, h[0]), __hmax2(__hmax2(h[1], h[2]), h[3]));
    }
    return fmaxf(__low2float(m2), __high2float(m2));
  }
};
template <> struct RowMax<__half> {
  static __device__ __forceinline__ float of(const uint4* row, int tid, int npk, int nt) {
    __half2 m2 = __float2half2_rn(-INFINITY);
#pragma unroll 4
    for (int pk = tid; pk < npk; pk += nt) {
      const uint4 raw = row[pk];
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      m2 = __hmax2(__hmax2(m2, h[0]), __hmax2(__hmax2(h[1], h[2]), h[3]));
    }
    return fmaxf(__low2float(m2), __high2float(m2));
  }
};

// The same computation with the rows staged in shared memory.  One persistent CTA per SM owns every gridDim.x-th row; a
// ring of whole rows (64 KB each for 32000 bfloat16 logits, three of them) is filled by bulk asynchronous copies that
// complete on mbarriers, so the next row is on its way from HBM while the two halves of the CTA sweep one row each, three
// times out of shared memory (max, sum of exponentials, gradient), and the gradients stream out.  Two rows at once because
// one row's sweeps are chains of shared-memory, special-function and barrier latencies that a single set of warps cannot fill.  The register-resident kernel above
// has nothing in flight while a block reduces and exponentiates; this one keeps the memory system busy throughout.
// Rows that do not count are never loaded.  Every wait is bounded: when one runs out the block marks the rows it has
// not finished with a NaN loss (which makes the mean loss NaN), lets its outstanding copies land (bounded too) and returns.
template <typename T, int NT>
__global__ void __launch_bounds__(NT, 1)
shifted_ce_staged_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ n_valid,
                         float* __restrict__ row_loss, T* d_logits, int B, int Tn, int V,
                         int64_t ls_b, int64_t ls_t, int64_t lab_b, int64_t lab_t, int64_t ignore_index,
                         int n_stages, uint32_t stage_bytes) {
  using namespace tc;
  constexpr int W = 16 / sizeof(T);
  constexpr int kGroups = 2, GT = NT / kGroups;          // the two halves of the CTA sweep two rows at the same time
  extern __shared__ __align__(128) unsigned char ce_smem[];
  __shared__ float buf[kGroups][2][GT / 32];
  __shared__ int abort_flag;
  __shared__ int last_req[4];                            // per stage: the last row that counts whose copy was requested
  uint64_t* full = reinterpret_cast<uint64_t*>(ce_smem + size_t(n_stages) * stage_bytes);
  const int tid = threadIdx.x, gid = tid / GT, gt = tid % GT;
  const float scale = 1.0f / fmaxf(n_valid[0], 1.0f);
  const int n_rows = B * Tn, npk = V / W;
  const uint32_t row_bytes = uint32_t(V) * sizeof(T);
  const int n_mine = int(blockIdx.x) < n_rows ? (n_rows - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < n_stages; ++i) { mbar_init(&full[i], 1); last_req[i] = -1; }
    mbar_fence_init();
  }
  __syncthreads();
  Guard g{&abort_flag, nullptr};
  auto target_of = [&](int i) -> int64_t {               // target of my i-th row, or -1 when the row does not count
    const int row = int(blockIdx.x) + i * int(gridDim.x);
    const int b = row / Tn, t = row - b * Tn;
    if (t + 1 >= Tn) return -1;
    const int64_t target = labels[b * lab_b + (t + 1) * lab_t];
    return (target != ignore_index && target >= 0 && target < V) ? target : -1;
  };
  // Rows that count use the stages of the ring in turn: the k-th of them goes through stage k % n_stages, and the group
  // that has finished with row k asks for row k + n_stages.  A group leader walks its own cursor over the rows to find it.
  int c_i = 0, c_k = 0;                                  // (leaders only) c_i: first row not yet passed, c_k: rows that count before it
  auto request = [&](int kk) {                           // copy the kk-th row that counts into its stage, if there is one
    while (c_i < n_mine) {
      if (target_of(c_i) >= 0) {
        if (c_k == kk) break;
        ++c_k;
      }
      ++c_i;
    }
    if (c_i >= n_mine || g.aborted()) return;           // (after a wait has run out nothing new is requested)
#ifdef FAT_TEST_CE_WITHHOLD_ROW
    if (kk == FAT_TEST_CE_WITHHOLD_ROW && blockIdx.x == 0) return;      // test builds: this copy never happens
#endif
    const int row = int(blockIdx.x) + c_i * int(gridDim.x);
    const int b = row / Tn, t = row - b * Tn;
    const int st = kk % n_stages;
    last_req[st] = kk;
    mbar_expect_tx(&full[st], row_bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(ce_smem + size_t(st) * stage_bytes)), "l"(reinterpret_cast<uint64_t>(logits + b * ls_b + t * ls_t)),
                   "r"(row_bytes), "r"(smem_u32(&full[st])) : "memory");
  };
  if (tid == 0) {
    for (int kk = 0; kk < n_stages; ++kk) request(kk);
    c_i = 0; c_k = 0;                                    // the walk for this group's own requests starts over
  }

  bool ok = true;
  int phase = 0;                                         // which half of this group's `buf` the next reduction uses
  auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + gid), "r"(GT) : "memory"); };
  // One barrier per group-wide reduction: consecutive reductions alternate between the two halves of `buf`, and a half
  // is not written again before a later barrier has been passed by every thread that read it.
  auto reduce = [&](float v, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float w = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, w) : v + w;
    }
    float* half = buf[gid][phase];
    phase ^= 1;
    if ((gt & 31) == 0) half[gt >> 5] = v;
    group_sync();
    float r = half[0];
#pragma unroll
    for (int w = 1; w < GT / 32; ++w) r = is_max ? fmaxf(r, half[w]) : r + half[w];
    return r;
  };
  int k = 0;                                             // rows that count, seen so far
  for (int i = 0; i < n_mine; ++i) {
    const int row = int(blockIdx.x) + i * int(gridDim.x);
    T* dx = d_logits ? d_logits + int64_t(row) * V : nullptr;
    const int64_t target = target_of(i);
    if (target < 0) {                                    // the groups take turns with the rows that only need zeros
      if ((i & 1) == gid) {
        if (dx) for (int pk = gt; pk < npk; pk += GT) reinterpret_cast<uint4*>(dx)[pk] = make_uint4(0u, 0u, 0u, 0u);
        if (gt == 0) row_loss[row] = 0.f;
      }
      continue;
    }
    const int my_k = k++;
    if ((my_k & 1) != gid) continue;                     // the other group's row
    const int st = my_k % n_stages;
    // (a wait that runs out does not leave the loop: every thread keeps passing the same barriers, the abort flag makes
    //  all later waits return at once, and the rows are marked after the loop)
    ok = g.wait(&full[st], (my_k / n_stages) & 1, 200) && ok;
    uint4* srow = reinterpret_cast<uint4*>(ce_smem + size_t(st) * stage_bytes);
    const int tgt = int(target);
    const float x_target = gt == 0 ? Elem<T>::to_c(reinterpret_cast<const T*>(srow)[tgt]) : 0.f;
    float m = RowMax<T>::of(srow, gt, npk, GT);
    m = reduce(m, true);
    const float off = m * kLog2e;
    // the exponentials are summed in float32 and put back over the row in the tensor dtype (values in [0, 1]): the
    // gradient sweep then needs no second exponential per element, at the price of one more rounding of the gradient
    // (2^-9 relative for bfloat16 against a bar of 2e-2)
    const f32x2 l2e2 = pk2(kLog2e, kLog2e), noff2 = pk2(-off, -off);
    float sum = 0.f;
#pragma unroll 4
    for (int pk = gt; pk < npk; pk += GT) {
      f32x2 x2[W / 2];
      Pairs<T>::get(srow[pk], x2);
      uint32_t back[W / 2];
#pragma unroll
      for (int j = 0; j < W / 2; ++j) {
        float a0, a1;
        upk2(fma2(x2[j], l2e2, noff2), a0, a1);
        const float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
        sum += e0 + e1;
        back[j] = Pairs<T>::pack(e0, e1);
      }
      if (dx) Pairs<T>::store(srow + pk, back);          // (each thread rewrites only the packs it reads)
    }
    sum = reduce(sum, false);
    if (dx) {
      const float inv = scale / sum;                     // softmax normaliser and 1/n_valid in one factor
      const f32x2 inv2 = pk2(inv, inv);
#pragma unroll 4
      for (int pk = gt; pk < npk; pk += GT) {
        f32x2 e2[W / 2];
        Pairs<T>::get(srow[pk], e2);
        uint32_t o[W / 2];
#pragma unroll
        for (int j = 0; j < W / 2; ++j) {
          float o0, o1;
          upk2(mul2(e2[j], inv2), o0, o1);
          o[j] = Pairs<T>::pack(o0, o1);
        }
        Pairs<T>::stream(dx + int64_t(pk) * W, o);
      }
      // the target's element, by the thread that has just stored its pack (so this store lands after that one)
      if (gt == (tgt / W) % GT) dx[tgt] = Elem<T>::from_c(Elem<T>::to_c(reinterpret_cast<const T*>(srow)[tgt]) * inv - scale);
    }
    if (gt == 0) row_loss[row] = m + logf(sum) - x_target;
    fence_async_smem();
    group_sync();                                        // the group is done with the row: its stage may be refilled
    if (gt == 0) request(my_k + n_stages);
  }
  if (__syncthreads_or(!ok)) {
    // a copy never arrived: say so through the losses, then let what was requested land before the block goes away
    if (tid == 0) {
      for (int r = 0; r < n_mine; ++r) row_loss[int(blockIdx.x) + r * int(gridDim.x)] = __int_as_float(0x7fc00000);
      for (int st = 0; st < n_stages; ++st)            // copies that were requested may still be on their way into this CTA
        if (last_req[st] >= 0)
          for (uint32_t spin = 0; spin < 16 && !mbar_try_wait(&full[st], (last_req[st] / n_stages) & 1); ++spin) {}
    }
  }
}

// x *= s[0] unless s[0] == 1 (the usual case: loss.backward() with no loss scaling), in which case nothing is touched
template <typename T>
__global__ void __launch_bounds__(256)
scale_unless_one_kernel(T* __restrict__ x, int64_t n, const float* __restrict__ s) {
  const float f = s[0];
  if (f == 1.0f) return;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    x[i] = Elem<T>::from_c(Elem<T>::to_c(x[i]) * f);
}

template <typename T>
int shifted_ce_t(const void* logits, const int64_t* labels, const float* n_valid, float* row_loss, void* d_logits,
                 int B, int Tn, int V, int64_t ls_b, int64_t ls_t, int64_t lab_b, int64_t lab_t, int64_t ignore_index,
                 cudaStream_t st) {
  constexpr int W = 16 / sizeof(T);
  const bool aligned = V % W == 0 && ls_b % W == 0 && ls_t % W == 0 && reinterpret_cast<uintptr_t>(logits) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(d_logits) % 16 == 0;      // (a null d_logits counts as aligned)
  const int64_t rows = int64_t(B) * Tn;
  const unsigned grid = unsigned(rows < 64 * int64_t(num_sms()) ? rows : 64 * int64_t(num_sms()));
  auto go = [&](auto kern, int threads) {
    kern<<<grid, threads, 0, st>>>((const T*)logits, labels, n_valid, row_loss, (T*)d_logits, B, Tn, V, ls_b, ls_t, lab_b, lab_t,
                                   ignore_index);
  };
  // rows staged in shared memory when at least two of them fit next to each other
  const uint32_t stage_bytes = (uint32_t(V) * sizeof(T) + 127u) & ~127u;
  const int n_stages = int((kCeSmemBytes - 256) / stage_bytes) < 4 ? int((kCeSmemBytes - 256) / stage_bytes) : 4;
  if constexpr (sizeof(T) == 2) if (FAT_CE_STAGED && aligned && n_stages >= 2 && rows >= 2 * int64_t(num_sms())) {
    const size_t smem = size_t(n_stages) * stage_bytes + 64;
    auto kern = shifted_ce_staged_kernel<T, kCeStagedThreads>;
    static bool configured = false;              // (per instantiation; racing threads set the same value)
    if (!configured) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kCeSmemBytes));
      configured = true;
    }
    kern<<<unsigned(num_sms()), kCeStagedThreads, smem, st>>>((const T*)logits, labels, n_valid, row_loss, (T*)d_logits, B, Tn, V, ls_b, ls_t,
                                                             lab_b, lab_t, ignore_index, n_stages, stage_bytes);
    return check_launch("shifted_ce_staged");
  }
  if (aligned && V / W <= 256 * kCePacks) go(shifted_ce_kernel<T, 256, true>, 256);
  else if (aligned && V / W <= 512 * kCePacks) go(shifted_ce_kernel<T, 512, true>, 512);
  else go(shifted_ce_kernel<T, 512, false>, 512);
  return check_launch("shifted_ce");
}

template <typename T>
int scale_t(void* x, int64_t n, const float* s, cudaStream_t st) {
  const int64_t blocks = (n + 255) / 256;
  scale_unless_one_kernel<T><<<unsigned(blocks < 16 * int64_t(num_sms()) ? blocks : 16 * int64_t(num_sms())), 256, 0, st>>>((T*)x, n, s);
  return check_launch("scale_unless_one");
}

}  // namespace
}  // namespace fat

using namespace fat;

extern "C" {

int fat_shifted_ce_fwd(const void* logits, const int64_t* labels, const float* n_valid, float* row_loss, void* d_logits,
                       int B, int T, int V, int64_t logits_batch_stride, int64_t logits_token_stride,
                       int64_t labels_batch_stride, int64_t labels_token_stride, int64_t ignore_index, int dtype,
                       void* stream) {
  if (B < 0 || T < 0 || V <= 0 || int64_t(B) * T > (int64_t(1) << 31) - 1) {
    set_error("shifted_ce_fwd: bad shape [%d, %d, %d]", B, T, V);
    return FAT_ERR_SHAPE;
  }
  if (B == 0 || T == 0) return FAT_OK;
  if (!logits || !labels || !n_valid || !row_loss) { set_error("shifted_ce_fwd: null pointer"); return FAT_ERR_NULL; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FAT_F32: return shifted_ce_t<float>(logits, labels, n_valid, row_loss, d_logits, B, T, V, logits_batch_stride,
                                             logits_token_stride, labels_batch_stride, labels_token_stride, ignore_index, st);
    case FAT_BF16: return shifted_ce_t<__nv_bfloat16>(logits, labels, n_valid, row_loss, d_logits, B, T, V, logits_batch_stride,
                                                      logits_token_stride, labels_batch_stride, labels_token_stride, ignore_index, st);
    case FAT_F16: return shifted_ce_t<__half>(logits, labels, n_valid, row_loss, d_logits, B, T, V, logits_batch_stride,
                                              logits_token_stride, labels_batch_stride, labels_token_stride, ignore_index, st);
    default: set_error("shifted_ce_fwd: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE;
  }
}

int fat_scale_unless_one(void* x, int64_t n, const float* scale, int dtype, void* stream) {
  if (n < 0) { set_error("scale_unless_one: bad size %lld", (long long)n); return FAT_ERR_SHAPE; }
  if (n == 0) return FAT_OK;
  if (!x || !scale) { set_error("scale_unless_one: null pointer"); return FAT_ERR_NULL; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FAT_F32: return scale_t<float>(x, n, scale, st);
    case FAT_BF16: return scale_t<__nv_bfloat16>(x, n, scale, st);
    case FAT_F16: return scale_t<__half>(x, n, scale, st);
    default: set_error("scale_unless_one: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE;
  }
}

}  // extern "C"
