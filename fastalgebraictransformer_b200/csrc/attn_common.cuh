// Argument block shared by the attention kernel families (SIMT and tcgen05).
#pragma once

#include "common.cuh"

namespace fat {

// Everything a rational-attention launch needs, passed by value to the kernels.
// Strides are in elements, {batch, head, token}; the head dimension has unit stride.
struct AttnParams {
  const void* q; const void* k; const void* v; const float* slopes;
  void* out; float* L;                        // forward outputs / backward inputs
  void* out_lo;                               // optional rounding residual of out (same strides), may be null
  const void* d_out; void* d_q; void* d_k; void* d_v;
  float* delta;                               // workspace: Delta_i = d_out_i . out_i, [B,H,T]
  float* dq_acc;                              // workspace: float32 d_q accumulator (tensor path)
  int B, H, T, D;
  int64_t qs[3], ks[3], vs[3], os[3], dos[3], dqs[3], dks[3], dvs[3];
  float scale, eps;
  int causal;
  int deterministic;                          // tensor path backward: two kernels without atomics instead of the fused one
  int* status;
  // optional padding mask over the keys: bit (j & 31) of key_mask[b * mask_words + (j >> 5)] set = key j of batch
  // element b takes part; mask_words = 4 * ceil(T / 128), bits from T on are clear.  Null: every key takes part.
  const uint32_t* key_mask;
  int mask_words;
};

// Whether key `col` (< T) of batch element b takes part.
__device__ __forceinline__ bool key_kept(const AttnParams& p, int b, int col) {
  return !p.key_mask || ((__ldg(p.key_mask + int64_t(b) * p.mask_words + (col >> 5)) >> (col & 31)) & 1u);
}

// SIMT family (attn_simt.cu)
int attn_fwd_simt(const AttnParams& p, int dtype, cudaStream_t st);
int attn_bwd_simt(const AttnParams& p, int dtype, cudaStream_t st);

// tcgen05 family (attn_tc_fwd.cu / attn_tc_bwd.cu)
bool   attn_tc_eligible(int T, int D, int dtype, bool aligned, bool causal, bool backward);
int    attn_fwd_tc(const AttnParams& p, int dtype, cudaStream_t st);
int    attn_bwd_tc(const AttnParams& p, int dtype, cudaStream_t st);
size_t attn_bwd_tc_workspace_bytes(int B, int H, int T, int D, int dtype);

}  // namespace fat
