// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is fetched from the
// driver at run time (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#include <mutex>
#include <unordered_map>

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

// A tensor map is a pure function of (address, extents, strides, box, element kind), and a training loop presents the
// same few of them step after step, so encoded maps are kept: a launch then costs a hash lookup per operand instead of
// a driver call.  The table is dropped wholesale when it grows past a bound (addresses from a caching allocator recur,
// so in practice it stays small).
struct MapKey {
  const void* base; int B, H, T, D, box_d, box_t, kind; int64_t s0, s1, s2;
  bool operator==(const MapKey& o) const {
    return base == o.base && B == o.B && H == o.H && T == o.T && D == o.D && box_d == o.box_d && box_t == o.box_t &&
           kind == o.kind && s0 == o.s0 && s1 == o.s1 && s2 == o.s2;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
    mix(reinterpret_cast<uintptr_t>(k.base)); mix(uint64_t(k.B) << 32 | uint32_t(k.H)); mix(uint64_t(k.T) << 32 | uint32_t(k.D));
    mix(uint64_t(k.box_d) << 40 | uint64_t(k.box_t) << 8 | uint32_t(k.kind)); mix(uint64_t(k.s0)); mix(uint64_t(k.s1)); mix(uint64_t(k.s2));
    return size_t(h);
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
constexpr size_t kMaxCachedMaps = 4096;

bool cached_map(const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) return false;
  *out = it->second;
  return true;
}
void remember_map(const MapKey& key, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lock(g_map_mu);
  if (g_maps.size() >= kMaxCachedMaps) g_maps.clear();
  g_maps.emplace(key, m);
}

}  // namespace

bool make_tmap_bhtd(CUtensorMap* out, const void* base, int B, int H, int T, int D,
                    const int64_t* s, int box_d, int box_t) {
  const MapKey key{base, B, H, T, D, box_d, box_t, 16, s[0], s[1], s[2]};
  if (cached_map(key, out)) return true;
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
  remember_map(key, *out);
  return true;
}

bool make_tmap_bhtd_f32(CUtensorMap* out, const void* base, int B, int H, int T, int D, int box_d, int box_t) {
  const MapKey key{base, B, H, T, D, box_d, box_t, 32, 0, 0, 0};
  if (cached_map(key, out)) return true;
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
  remember_map(key, *out);
  return true;
}

}  // namespace fat
