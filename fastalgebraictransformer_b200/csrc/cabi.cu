// The C ABI: argument validation, path selection and error reporting around the kernels.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "attn_common.cuh"

namespace fat {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};

// Called exactly once after every kernel launch of this library.
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) { g_launches.fetch_add(1, std::memory_order_relaxed); return FAT_OK; }
  set_error("%s: %s", what, cudaGetErrorString(e));
  return FAT_ERR_LAUNCH;
}

int num_sms() {
  constexpr int kMaxDev = 64;
  static std::atomic<int> cached[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// The tensor-core attention kernels cover 16-bit tensors, head sizes 64 and 128 (causal or not), and pointers /
// strides that TMA can address (16-byte aligned, strides multiples of 8 elements).
bool attn_tc_eligible(int T, int D, int dtype, bool aligned, bool causal, bool backward) {
  (void)backward; (void)causal;
  return T >= 1 && (D == 64 || D == 128) && (dtype == FAT_BF16 || dtype == FAT_F16) && aligned;
}

namespace {

bool strides_aligned(const int64_t* s, int w) { return s[0] % w == 0 && s[1] % w == 0 && s[2] % w == 0; }

int check_attn_shape(const char* what, int B, int H, int T, int D) {
  if (B < 0 || H <= 0 || T < 0 || D <= 0) {
    set_error("%s: bad shape [B=%d, H=%d, T=%d, D=%d]", what, B, H, T, D);
    return FAT_ERR_SHAPE;
  }
  if (H > 65535 || B > 65535) {
    set_error("%s: B and H must not exceed 65535", what);
    return FAT_ERR_UNSUPPORTED;
  }
  return FAT_OK;
}

void copy3(int64_t (&dst)[3], const int64_t* src) { dst[0] = src[0]; dst[1] = src[1]; dst[2] = src[2]; }

// Resolves the kernel family.  Returns FAT_PATH_SIMT / FAT_PATH_TENSOR, or a negative status.
int resolve_path(const char* what, int path, int T, int D, int dtype, bool aligned, bool causal, bool backward) {
  const bool ok = attn_tc_eligible(T, D, dtype, aligned, causal, backward);
  if (path == FAT_PATH_SIMT) return FAT_PATH_SIMT;
  if (path == FAT_PATH_TENSOR || path == FAT_PATH_TENSOR_DETERMINISTIC) {
    if (!ok) {
      set_error("%s: the tensor-core path needs bf16/f16, D in {64,128}, 16-byte aligned pointers and "
                "strides (got dtype %d, D=%d, aligned=%d)", what, dtype, D, int(aligned));
      return aligned ? -FAT_ERR_UNSUPPORTED : -FAT_ERR_ALIGNMENT;
    }
    return FAT_PATH_TENSOR;
  }
  if (path != FAT_PATH_AUTO) { set_error("%s: unknown path selector %d", what, path); return -FAT_ERR_UNSUPPORTED; }
  return ok ? FAT_PATH_TENSOR : FAT_PATH_SIMT;
}

}  // namespace
}  // namespace fat

using namespace fat;


extern "C" {

int fat_version(void) { return 100; }

const char* fat_last_error(void) { return g_err; }

unsigned long long fat_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* fat_error_string(int code) {
  switch (code) {
    case FAT_OK: return "ok";
    case FAT_ERR_DTYPE: return "unsupported dtype";
    case FAT_ERR_SHAPE: return "bad shape";
    case FAT_ERR_UNSUPPORTED: return "unsupported configuration";
    case FAT_ERR_ALIGNMENT: return "misaligned pointer or stride";
    case FAT_ERR_WORKSPACE: return "workspace missing or too small";
    case FAT_ERR_LAUNCH: return "CUDA launch failed";
    case FAT_ERR_NULL: return "null pointer";
    default: return "unknown error code";
  }
}

int fat_attn_select_path(int T, int D, int dtype, int aligned, int causal, int backward) {
  return attn_tc_eligible(T, D, dtype, aligned != 0, causal != 0, backward != 0) ? FAT_PATH_TENSOR : FAT_PATH_SIMT;
}

int fat_attn_fwd(const void* q, const void* k, const void* v, const float* slopes, void* out, void* out_lo, float* L,
                 int B, int H, int T, int D,
                 const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os,
                 double scale, double eps, int causal, int dtype, int path, int* status, void* stream) {
  return fat_attn_fwd_masked(q, k, v, slopes, nullptr, out, out_lo, L, B, H, T, D, qs, ks, vs, os, scale, eps, causal, dtype, path,
                             status, stream);
}

int fat_attn_fwd_masked(const void* q, const void* k, const void* v, const float* slopes, const uint32_t* key_mask_bits,
                        void* out, void* out_lo, float* L, int B, int H, int T, int D,
                        const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os,
                        double scale, double eps, int causal, int dtype, int path, int* status, void* stream) {
  if (int rc = check_attn_shape("attn_fwd", B, H, T, D)) return rc;
  if (dtype != FAT_F32 && dtype != FAT_BF16 && dtype != FAT_F16) { set_error("attn_fwd: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE; }
  if (B == 0 || T == 0) return FAT_OK;
  if (!q || !k || !v || !slopes || !out || !L || !qs || !ks || !vs || !os) { set_error("attn_fwd: null pointer"); return FAT_ERR_NULL; }
  const int w = dtype == FAT_F32 ? 4 : 8;
  const bool aligned = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(out_lo) &&
                       strides_aligned(qs, w) && strides_aligned(ks, w) && strides_aligned(vs, w) && strides_aligned(os, w);
  const int sel = resolve_path("attn_fwd", path, T, D, dtype, aligned, causal != 0, false);
  if (sel < 0) return -sel;
  AttnParams p{};
  p.q = q; p.k = k; p.v = v; p.slopes = slopes; p.out = out; p.out_lo = out_lo; p.L = L;
  p.B = B; p.H = H; p.T = T; p.D = D;
  copy3(p.qs, qs); copy3(p.ks, ks); copy3(p.vs, vs); copy3(p.os, os);
  p.scale = float(scale); p.eps = float(eps); p.causal = causal != 0; p.status = status;
  p.key_mask = key_mask_bits; p.mask_words = fat_key_mask_words(T);
  return sel == FAT_PATH_TENSOR ? attn_fwd_tc(p, dtype, (cudaStream_t)stream) : attn_fwd_simt(p, dtype, (cudaStream_t)stream);
}

size_t fat_attn_bwd_workspace_bytes(int B, int H, int T, int D, int dtype, int path) {
  if (B <= 0 || H <= 0 || T <= 0 || D <= 0) return 0;
  const size_t delta = size_t(B) * H * T * sizeof(float);
  const bool tc = path != FAT_PATH_SIMT && attn_tc_eligible(T, D, dtype, true, true, true);
  return tc ? attn_bwd_tc_workspace_bytes(B, H, T, D, dtype) : delta;
}

int fat_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* out_lo, const float* L,
                 const void* d_out, const float* slopes, void* d_q, void* d_k, void* d_v,
                 void* workspace, size_t workspace_bytes, int B, int H, int T, int D,
                 const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, const int64_t* dos,
                 const int64_t* dqs, const int64_t* dks, const int64_t* dvs,
                 double scale, double eps, int causal, int dtype, int path, int* status, void* stream) {
  return fat_attn_bwd_masked(q, k, v, out, out_lo, L, d_out, slopes, nullptr, d_q, d_k, d_v, workspace, workspace_bytes, B, H, T, D,
                             qs, ks, vs, os, dos, dqs, dks, dvs, scale, eps, causal, dtype, path, status, stream);
}

int fat_attn_bwd_masked(const void* q, const void* k, const void* v, const void* out, const void* out_lo, const float* L,
                        const void* d_out, const float* slopes, const uint32_t* key_mask_bits, void* d_q, void* d_k, void* d_v,
                        void* workspace, size_t workspace_bytes, int B, int H, int T, int D,
                        const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, const int64_t* dos,
                        const int64_t* dqs, const int64_t* dks, const int64_t* dvs,
                        double scale, double eps, int causal, int dtype, int path, int* status, void* stream) {
  if (int rc = check_attn_shape("attn_bwd", B, H, T, D)) return rc;
  if (dtype != FAT_F32 && dtype != FAT_BF16 && dtype != FAT_F16) { set_error("attn_bwd: unsupported dtype tag %d", dtype); return FAT_ERR_DTYPE; }
  if (B == 0 || T == 0) return FAT_OK;
  if (!q || !k || !v || !out || !L || !d_out || !slopes || !d_q || !d_k || !d_v ||
      !qs || !ks || !vs || !os || !dos || !dqs || !dks || !dvs) { set_error("attn_bwd: null pointer"); return FAT_ERR_NULL; }
  const int w = dtype == FAT_F32 ? 4 : 8;
  const bool aligned = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(out_lo) && aligned16(d_out) &&
                       aligned16(d_q) && aligned16(d_k) && aligned16(d_v) &&
                       strides_aligned(qs, w) && strides_aligned(ks, w) && strides_aligned(vs, w) && strides_aligned(os, w) &&
                       strides_aligned(dos, w) && strides_aligned(dqs, w) && strides_aligned(dks, w) && strides_aligned(dvs, w);
  const int sel = resolve_path("attn_bwd", path, T, D, dtype, aligned, causal != 0, true);
  if (sel < 0) return -sel;
  const size_t need = sel == FAT_PATH_TENSOR ? attn_bwd_tc_workspace_bytes(B, H, T, D, dtype) : size_t(B) * H * T * sizeof(float);
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) {
    set_error("attn_bwd: workspace of %zu bytes (16-byte aligned) required, got %zu at %p", need, workspace_bytes, workspace);
    return FAT_ERR_WORKSPACE;
  }
  AttnParams p{};
  p.q = q; p.k = k; p.v = v; p.slopes = slopes; p.out = const_cast<void*>(out); p.out_lo = const_cast<void*>(out_lo); p.L = const_cast<float*>(L);
  p.d_out = d_out; p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  p.delta = static_cast<float*>(workspace);
  p.dq_acc = static_cast<float*>(workspace) + ((size_t(B) * H * T + 3) / 4) * 4;
  p.B = B; p.H = H; p.T = T; p.D = D;
  copy3(p.qs, qs); copy3(p.ks, ks); copy3(p.vs, vs); copy3(p.os, os); copy3(p.dos, dos);
  copy3(p.dqs, dqs); copy3(p.dks, dks); copy3(p.dvs, dvs);
  p.scale = float(scale); p.eps = float(eps); p.causal = causal != 0; p.status = status;
  p.deterministic = path == FAT_PATH_TENSOR_DETERMINISTIC;
  p.key_mask = key_mask_bits; p.mask_words = fat_key_mask_words(T);
  return sel == FAT_PATH_TENSOR ? attn_bwd_tc(p, dtype, (cudaStream_t)stream) : attn_bwd_simt(p, dtype, (cudaStream_t)stream);
}

}  // extern "C"
