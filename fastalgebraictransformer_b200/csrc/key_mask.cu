// Padding mask over the keys, packed to one bit per key for the attention kernels.
//
// The reference's model takes `attention_mask` [B, T] (0 = padding) and fills the scores of padded keys with -1e4 on its
// PyTorch path (algebraic_model.py:128-131: `scores.masked_fill_(mask[:, None, None, :] == 0, -1e4)`); its Triton path
// ignores the mask (algebraic_model.py:93-104).  The attention kernels here take the mask as bits: word w of batch
// element b covers keys 32 w .. 32 w + 31, bit set = the key takes part, 4 * ceil(T / 128) words per batch element so that
// every 128-key tile owns four whole words, bits from T on clear (a ragged last tile needs no other treatment).
#include <cstdint>

#include "attn_common.cuh"

namespace fat {
namespace {

__global__ void __launch_bounds__(256)
pack_key_mask_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ bits, int B, int T, int words,
                     int64_t batch_stride, int64_t token_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t n_words = int64_t(B) * words;
  for (int64_t w = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < n_words; w += (int64_t(gridDim.x) * blockDim.x) >> 5) {
    const int b = int(w / words), j = int(w % words) * 32 + lane;
    const bool keep = j < T && mask[b * batch_stride + j * token_stride] != 0;
    const uint32_t word = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) bits[w] = word;
  }
}

}  // namespace
}  // namespace fat

using namespace fat;

extern "C" int fat_key_mask_words(int T) { return T > 0 ? 4 * ((T + 127) / 128) : 0; }

extern "C" int fat_pack_key_mask(const uint8_t* mask, uint32_t* bits, int B, int T, int64_t mask_batch_stride,
                                 int64_t mask_token_stride, void* stream) {
  if (B < 0 || T < 0) { set_error("pack_key_mask: bad shape [%d, %d]", B, T); return FAT_ERR_SHAPE; }
  if (B == 0 || T == 0) return FAT_OK;
  if (!mask || !bits) { set_error("pack_key_mask: null pointer"); return FAT_ERR_NULL; }
  const int words = fat_key_mask_words(T);
  const int64_t warps = int64_t(B) * words;
  const int64_t blocks = (warps + 7) / 8;
  pack_key_mask_kernel<<<unsigned(blocks < 8 * int64_t(num_sms()) ? blocks : 8 * int64_t(num_sms())), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, bits, B, T, words, mask_batch_stride, mask_token_stride);
  return check_launch("pack_key_mask");
}
