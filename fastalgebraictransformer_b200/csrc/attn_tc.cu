// Eligibility of the tcgen05 attention kernels.
#include "attn_common.cuh"
namespace fat {
// The tensor-core kernels cover 16-bit tensors, head sizes 64 and 128, causal masking, and
// pointers / strides that TMA can address (16-byte aligned, strides multiples of 8 elements).
bool attn_tc_eligible(int T, int D, int dtype, bool aligned, bool causal, bool backward) {
  (void)backward;
  return T >= 1 && (D == 64 || D == 128) && (dtype == FAT_BF16 || dtype == FAT_F16) && aligned && causal;
}
}
