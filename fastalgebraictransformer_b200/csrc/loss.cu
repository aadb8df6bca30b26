// Shifted cross-entropy of the language-model head in one pass over the logits.
//
// The reference computes  F.cross_entropy(logits[..., :-1, :].contiguous().view(-1, V), labels[..., 1:].view(-1),
// ignore_index=-100)  (algebraic_model.py:229-235): a copy of the logits, a log-softmax pass that writes a tensor of the
// same size, and in the backward a log-softmax-backward pass and a zero-padded slice gradient.  Here one kernel reads
// every logits row once, keeps it in registers, and writes the row's loss and the row of d(loss)/d(logits) (already
// divided by the number of valid targets; zero for the last position of a sequence and for ignored targets).  The
// backward only multiplies by the incoming scalar gradient, and skips even that when the scalar is 1.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "../../include/fat_b200.h"
#include "common.cuh"

namespace fat {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kCePacks = 16;                       // 16-byte packs of one row a thread keeps in registers

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
