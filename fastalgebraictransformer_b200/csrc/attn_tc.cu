// Eligibility of the tcgen05 attention kernels and (until it lands) the backward placeholder.
#include "attn_common.cuh"
namespace fat {
// The tensor-core kernels cover 16-bit tensors, head sizes 64 and 128, causal masking, and
// pointers / strides that TMA can address (16-byte aligned, strides multiples of 8 elements).
bool attn_tc_eligible(int T, int D, int dtype, bool aligned, bool causal, bool backward) {
  if (backward) return false;
  return T >= 1 && (D == 64 || D == 128) && (dtype == FAT_BF16 || dtype == FAT_F16) && aligned && causal;
}
int attn_bwd_tc(const AttnParams&, int, cudaStream_t) { set_error("tensor-core backward is not built"); return FAT_ERR_UNSUPPORTED; }
size_t attn_bwd_tc_workspace_bytes(int B, int H, int T, int D) { return size_t(B) * H * T * 4; }
}
