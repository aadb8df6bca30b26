// placeholder until the tcgen05 kernels land
#include "attn_common.cuh"
namespace fat {
bool attn_tc_eligible(int, int, int, bool) { return false; }
int attn_fwd_tc(const AttnParams&, int, cudaStream_t) { set_error("tensor path not built"); return FAT_ERR_UNSUPPORTED; }
int attn_bwd_tc(const AttnParams&, int, cudaStream_t) { set_error("tensor path not built"); return FAT_ERR_UNSUPPORTED; }
size_t attn_bwd_tc_workspace_bytes(int B, int H, int T, int D) { return size_t(B) * H * T * 4; }
}
