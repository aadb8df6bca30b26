// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is fetched from the
// driver at run time (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace fat {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

}  // namespace

bool make_tmap_bhtd(CUtensorMap* out, const void* base, int B, int H, int T, int D,
                    const int64_t* s, int box_d, int box_t) {
  // The encoder is a driver-API call: it needs the primary context bound to the calling thread,
  // which a thread that has only been handed pointers (e.g. an autograd worker) may not have yet.
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  EncodeFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return false; }
  const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(T), cuuint64_t(H), cuuint64_t(B)};
  // byte strides of dims 1..3; a dimension of extent 1 may carry any stride, give it a legal one
  auto bytes = [](int64_t elems, int extent, int64_t fallback) {
    return cuuint64_t((extent > 1 ? elems : fallback) * 2);
  };
  const cuuint64_t strides[3] = {bytes(s[2], T, D), bytes(s[1], H, int64_t(D) * T), bytes(s[0], B, int64_t(D) * T * H)};
  const cuuint32_t box[4] = {cuuint32_t(box_d), cuuint32_t(box_t), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (dims %d,%d,%d,%d strides %lld,%lld,%lld box %d,%d)", int(r),
              D, T, H, B, (long long)strides[0], (long long)strides[1], (long long)strides[2], box_d, box_t);
    return false;
  }
  return true;
}

bool make_tmap_bhtd_f32(CUtensorMap* out, const void* base, int B, int H, int T, int D, int box_d, int box_t) {
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  EncodeFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return false; }
  const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(T), cuuint64_t(H), cuuint64_t(B)};
  const cuuint64_t strides[3] = {cuuint64_t(D) * 4, cuuint64_t(D) * T * 4, cuuint64_t(D) * T * H * 4};
  const cuuint32_t box[4] = {cuuint32_t(box_d), cuuint32_t(box_t), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (float32) failed with code %d (dims %d,%d,%d,%d box %d,%d)", int(r), D, T, H, B, box_d, box_t);
    return false;
  }
  return true;
}

}  // namespace fat
