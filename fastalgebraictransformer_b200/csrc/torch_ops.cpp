// torch.library operators of the `algebraic` namespace, registered from C++.
//
// Each operator allocates its outputs with ATen, takes raw pointers / element strides / the current CUDA stream of
// its tensors and calls the C ABI of libfat_b200.so (include/fat_b200.h); a non-zero return code becomes a
// c10::Error (RuntimeError in Python).  Nothing here launches a kernel of its own.  Shape functions for meta
// tensors and the autograd formulas are registered from Python (ops.py) on these same operators.
//
// Built by `python -m fastalgebraictransformer_b200.build` into libfat_torch_ops.so next to libfat_b200.so.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <array>
#include <mutex>
#include <tuple>

#include "../../include/fat_b200.h"

namespace {

using at::Tensor;

void check(int rc) {
  TORCH_CHECK(rc == 0, "libfat_b200: ", fat_error_string(rc), " — ", fat_last_error());
}

int dtype_tag(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return FAT_F32;
    case at::kBFloat16: return FAT_BF16;
    case at::kHalf: return FAT_F16;
    case at::kDouble: return FAT_F64;
    default: TORCH_CHECK_TYPE(false, "unsupported dtype ", t.scalar_type());
  }
}

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void cuda_check(std::initializer_list<const Tensor*> ts) {
  const Tensor* first = *ts.begin();
  for (const Tensor* t : ts) {
    TORCH_CHECK(t->is_cuda(), "algebraic ops run on CUDA tensors only (there is no CPU fallback)");
    TORCH_CHECK(t->device() == first->device(), "all tensors must be on the same device");
  }
}

// View `t` as [n_rows, n_cols] with unit column stride, copying only when it must: a slice of the last dimension of
// a dense tensor (one half of chunk(2, -1)) has equally spaced rows, so (n_rows, row_stride) describes it in place.
Tensor rows(const Tensor& t) {
  const int64_t n = t.size(-1);
  if (t.dim() == 2 && t.stride(1) == 1) return t;
  if (t.is_contiguous()) return t.view({-1, n});
  if (t.stride(-1) == 1 || n == 1) {
    const int64_t st = t.dim() >= 2 ? t.stride(-2) : n;
    bool ok = true;
    int64_t expect = st;
    for (int64_t d = t.dim() - 2; d >= 0; --d) {
      if (t.size(d) != 1 && t.stride(d) != expect) { ok = false; break; }
      expect = t.stride(d) * t.size(d);
    }
    if (ok && n > 0) return t.as_strided({t.numel() / n, n}, {st, 1}, t.storage_offset());
  }
  return t.contiguous().view({-1, n});
}

std::array<int64_t, 3> strides3(const Tensor& t) { return {t.stride(0), t.stride(1), t.stride(2)}; }

// ------------------------------------------------------------------------------------- device status word
// One int32 per device that the attention kernels write when a bounded wait runs out or an operand leaves float16's
// range; Python reads (and clears) it through algebraic::device_status.
Tensor status_word(int device) {
  static std::mutex mu;
  static std::array<Tensor, 64> words;
  TORCH_CHECK(device >= 0 && device < 64, "device index out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!words[device].defined())
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return words[device];
}

Tensor device_status(int64_t device) { return status_word(int(device)); }

// ------------------------------------------------------------------------------------- SwiGLU
Tensor swiglu_fwd(const Tensor& gate, const Tensor& value) {
  cuda_check({&gate, &value});
  TORCH_CHECK(gate.sizes() == value.sizes() && gate.scalar_type() == value.scalar_type(), "gate and value must match");
  Tensor out = at::empty(gate.sizes(), gate.options());
  if (gate.numel() == 0) return out;
  const Tensor g = rows(gate), v = rows(value), o = out.view({-1, gate.size(-1)});
  c10::cuda::CUDAGuard guard(gate.device());
  check(fat_swiglu_fwd(g.data_ptr(), v.data_ptr(), o.data_ptr(), g.size(0), g.size(1), g.stride(0), v.stride(0), o.stride(0),
                       dtype_tag(gate), stream_of(gate)));
  return out;
}

std::tuple<Tensor, Tensor> swiglu_bwd(const Tensor& d_out, const Tensor& gate, const Tensor& value) {
  cuda_check({&d_out, &gate, &value});
  const int64_t n = gate.size(-1);
  // both gradients live in one [rows, 2n] buffer: when gate/value were the two halves of a packed projection,
  // autograd's concatenation of the halves becomes a no-op copy target of the same layout
  auto shape = gate.sizes().vec();
  shape.back() = 2 * n;
  Tensor packed = at::empty(shape, gate.options());
  Tensor d_gate = packed.narrow(-1, 0, n), d_value = packed.narrow(-1, n, n);
  if (gate.numel() == 0) return {d_gate, d_value};
  const Tensor go = rows(d_out), g = rows(gate), v = rows(value), dg = rows(d_gate), dv = rows(d_value);
  c10::cuda::CUDAGuard guard(gate.device());
  check(fat_swiglu_bwd(go.data_ptr(), g.data_ptr(), v.data_ptr(), dg.data_ptr(), dv.data_ptr(), g.size(0), n, go.stride(0),
                       g.stride(0), v.stride(0), dg.stride(0), dv.stride(0), dtype_tag(gate), stream_of(gate)));
  return {d_gate, d_value};
}

// ------------------------------------------------------------------------------------- mean-error norm
std::tuple<Tensor, Tensor> norm_fwd(const Tensor& x, const Tensor& weight, double eps) {
  cuda_check({&x, &weight});
  const int64_t n = x.size(-1);
  TORCH_CHECK(weight.dim() == 1 && weight.size(0) == n, "weight must be [n_cols]");
  const Tensor w = weight.to(x.scalar_type()).contiguous();
  Tensor y = at::empty(x.sizes(), x.options());
  const Tensor xr = rows(x);
  Tensor mean = at::empty({xr.size(0)}, x.options().dtype(at::kFloat));
  if (x.numel()) {
    const Tensor yr = y.view({-1, n});
    c10::cuda::CUDAGuard guard(x.device());
    check(fat_norm_fwd(xr.data_ptr(), w.data_ptr(), yr.data_ptr(), mean.data_ptr<float>(), xr.size(0), n, xr.stride(0),
                       yr.stride(0), eps, dtype_tag(x), stream_of(x)));
  }
  return {y, mean};
}

std::tuple<Tensor, Tensor> norm_bwd(const Tensor& d_out, const Tensor& x, const Tensor& weight, const Tensor& mean, double eps) {
  cuda_check({&d_out, &x, &weight, &mean});
  const int64_t n = x.size(-1);
  const Tensor w = weight.to(x.scalar_type()).contiguous();
  Tensor d_x = at::empty(x.sizes(), x.options()), d_w = at::empty({n}, x.options());
  const Tensor go = rows(d_out), xr = rows(x), dxr = d_x.view({-1, n});
  const int tag = dtype_tag(x);
  c10::cuda::CUDAGuard guard(x.device());
  const size_t ws_bytes = fat_norm_bwd_workspace_bytes(xr.size(0), n, tag);
  Tensor ws = at::empty({int64_t(ws_bytes)}, x.options().dtype(at::kByte));
  check(fat_norm_bwd(go.data_ptr(), xr.data_ptr(), w.data_ptr(), mean.data_ptr<float>(), dxr.data_ptr(), d_w.data_ptr(),
                     ws.data_ptr(), ws_bytes, xr.size(0), n, go.numel() ? go.stride(0) : n, xr.numel() ? xr.stride(0) : n, n,
                     eps, tag, stream_of(x)));
  return {d_x, d_w.to(weight.scalar_type())};
}

// h = x + residual, y = mean_error_norm(h, weight), in one pass.  Returns (h, y, mean).
std::tuple<Tensor, Tensor, Tensor> add_norm_fwd(const Tensor& x, const Tensor& residual, const Tensor& weight, double eps) {
  cuda_check({&x, &residual, &weight});
  TORCH_CHECK(x.sizes() == residual.sizes() && x.scalar_type() == residual.scalar_type(), "x and residual must match");
  const int64_t n = x.size(-1);
  TORCH_CHECK(weight.dim() == 1 && weight.size(0) == n, "weight must be [n_cols]");
  const Tensor w = weight.to(x.scalar_type()).contiguous();
  Tensor h = at::empty(x.sizes(), x.options()), y = at::empty(x.sizes(), x.options());
  const Tensor xr = rows(x), rr = rows(residual);
  Tensor mean = at::empty({xr.size(0)}, x.options().dtype(at::kFloat));
  if (x.numel()) {
    const Tensor hr = h.view({-1, n}), yr = y.view({-1, n});
    c10::cuda::CUDAGuard guard(x.device());
    check(fat_add_norm_fwd(xr.data_ptr(), rr.data_ptr(), w.data_ptr(), hr.data_ptr(), yr.data_ptr(), mean.data_ptr<float>(),
                           xr.size(0), n, xr.stride(0), rr.stride(0), n, n, eps, dtype_tag(x), stream_of(x)));
  }
  return {h, y, mean};
}

// Gradient of the sum (shared by x and residual) and of the weight.
std::tuple<Tensor, Tensor> add_norm_bwd(const Tensor& d_y, const c10::optional<Tensor>& d_h, const Tensor& h, const Tensor& weight,
                                        const Tensor& mean, double eps) {
  cuda_check({&d_y, &h, &weight, &mean});
  const int64_t n = h.size(-1);
  const Tensor w = weight.to(h.scalar_type()).contiguous();
  Tensor d_sum = at::empty(h.sizes(), h.options()), d_w = at::empty({n}, h.options());
  const Tensor go = rows(d_y), hr = rows(h), dsr = d_sum.view({-1, n});
  Tensor dh;
  if (d_h.has_value() && d_h->defined()) dh = rows(d_h->to(h.scalar_type()));
  const bool has_dh = dh.defined() && dh.numel() > 0;
  const int tag = dtype_tag(h);
  c10::cuda::CUDAGuard guard(h.device());
  const size_t ws_bytes = fat_norm_bwd_workspace_bytes(hr.size(0), n, tag);
  Tensor ws = at::empty({int64_t(ws_bytes)}, h.options().dtype(at::kByte));
  check(fat_add_norm_bwd(go.data_ptr(), has_dh ? dh.data_ptr() : nullptr, hr.data_ptr(), w.data_ptr(), mean.data_ptr<float>(),
                         dsr.data_ptr(), d_w.data_ptr(), ws.data_ptr(), ws_bytes, hr.size(0), n, go.numel() ? go.stride(0) : n,
                         has_dh ? dh.stride(0) : n, hr.numel() ? hr.stride(0) : n, n, eps, tag, stream_of(h)));
  return {d_sum, d_w.to(weight.scalar_type())};
}

// ------------------------------------------------------------------------------------- loss head
Tensor count_valid(const Tensor& labels, int64_t ignore_index, int64_t V) {
  const Tensor counted = labels.slice(1, 1);
  return ((counted != ignore_index) & (counted >= 0) & (counted < V)).sum().to(at::kFloat).reshape({1});
}

// (loss, d_logits) of mean cross-entropy between logits[:, :-1] and labels[:, 1:]
std::tuple<Tensor, Tensor> shifted_ce_fwd(const Tensor& logits_in, const Tensor& labels, int64_t ignore_index) {
  cuda_check({&logits_in, &labels});
  TORCH_CHECK(logits_in.dim() == 3 && labels.dim() == 2 && labels.size(0) == logits_in.size(0) && labels.size(1) == logits_in.size(1) &&
              labels.scalar_type() == at::kLong, "logits [B,T,V] and int64 labels [B,T] expected");
  const Tensor logits = logits_in.stride(2) == 1 ? logits_in : logits_in.contiguous();
  const int64_t B = logits.size(0), T = logits.size(1), V = logits.size(2);
  const Tensor n_valid = count_valid(labels, ignore_index, V);
  Tensor row_loss = at::empty({B * T}, logits.options().dtype(at::kFloat));
  Tensor d_logits = at::empty({B, T, V}, logits.options());
  if (logits.numel()) {
    c10::cuda::CUDAGuard guard(logits.device());
    check(fat_shifted_ce_fwd(logits.data_ptr(), labels.data_ptr<int64_t>(), n_valid.data_ptr<float>(), row_loss.data_ptr<float>(),
                             d_logits.data_ptr(), int(B), int(T), int(V), logits.stride(0), logits.stride(1), labels.stride(0),
                             labels.stride(1), ignore_index, dtype_tag(logits), stream_of(logits)));
    return {row_loss.sum() / n_valid.clamp_min(1.0).squeeze(0), d_logits};
  }
  return {row_loss.sum(), d_logits};
}

// Loss head without the [B, T, V] logits: (loss, d_y, d_weight) of the mean cross-entropy between (y @ weight^T)[:, :-1]
// and labels[:, 1:].  The logits exist one sequence at a time: a [T, V] buffer is filled by the head GEMM, the loss kernel
// turns it in place into its own gradient, and two more GEMMs fold that gradient into d_y and d_weight before the buffer
// is reused.  want_grads = false: only the loss (d_y and d_weight come back empty).
std::tuple<Tensor, Tensor, Tensor> head_shifted_ce(const Tensor& y_in, const Tensor& weight, const Tensor& labels,
                                                   int64_t ignore_index, bool want_grads) {
  cuda_check({&y_in, &weight, &labels});
  TORCH_CHECK(y_in.dim() == 3 && weight.dim() == 2 && y_in.size(2) == weight.size(1) && labels.dim() == 2 &&
              labels.size(0) == y_in.size(0) && labels.size(1) == y_in.size(1), "y [B,T,C], weight [V,C], labels [B,T] expected");
  TORCH_CHECK(labels.scalar_type() == at::kLong && y_in.scalar_type() == weight.scalar_type(), "int64 labels; y and weight of one dtype");
  const Tensor y = y_in.contiguous();
  const int64_t B = y.size(0), T = y.size(1), V = weight.size(0);
  const Tensor n_valid = count_valid(labels, ignore_index, V);
  Tensor row_loss = at::zeros({B * T}, y.options().dtype(at::kFloat));
  Tensor d_y = want_grads ? at::empty_like(y) : at::empty({0}, y.options());
  Tensor d_w = want_grads ? at::empty_like(weight) : at::empty({0}, y.options());
  if (y.numel() && V) {
    Tensor buf = at::empty({T, V}, y.options());
    const Tensor wt = weight.t();
    const int tag = dtype_tag(y);
    c10::cuda::CUDAGuard guard(y.device());
    for (int64_t b = 0; b < B; ++b) {
      const Tensor yb = y.select(0, b);
      at::mm_out(buf, yb, wt);
      check(fat_shifted_ce_fwd(buf.data_ptr(), labels.select(0, b).data_ptr<int64_t>(), n_valid.data_ptr<float>(),
                               row_loss.data_ptr<float>() + b * T, want_grads ? buf.data_ptr() : nullptr, 1, int(T), int(V), T * V, V,
                               labels.stride(0), labels.stride(1), ignore_index, tag, stream_of(y)));
      if (want_grads) {
        Tensor dyb = d_y.select(0, b);
        at::mm_out(dyb, buf, weight);
        if (b == 0) at::mm_out(d_w, buf.t(), yb);
        else d_w.addmm_(buf.t(), yb);
      }
    }
  } else if (want_grads) {
    d_w.zero_();
  }
  return {row_loss.sum() / n_valid.clamp_min(1.0).squeeze(0), d_y, d_w};
}

void scale_unless_one(Tensor x, const Tensor& scale) {
  cuda_check({&x, &scale});
  TORCH_CHECK(x.is_contiguous() && scale.scalar_type() == at::kFloat && scale.numel() == 1, "contiguous x and a float32 scalar expected");
  if (x.numel() == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  check(fat_scale_unless_one(x.data_ptr(), x.numel(), scale.data_ptr<float>(), dtype_tag(x), stream_of(x)));
}

// ------------------------------------------------------------------------------------- rational softmax
Tensor softmax_fwd(const Tensor& x, double eps) {
  cuda_check({&x});
  const int64_t n = x.size(-1);
  Tensor p = at::empty(x.sizes(), x.options());
  if (x.numel()) {
    const Tensor xr = rows(x), pr = p.view({-1, n});
    c10::cuda::CUDAGuard guard(x.device());
    check(fat_softmax_fwd(xr.data_ptr(), pr.data_ptr(), xr.size(0), n, xr.stride(0), pr.stride(0), eps, dtype_tag(x), stream_of(x)));
  }
  return p;
}

Tensor softmax_bwd(const Tensor& d_out, const Tensor& x, double eps) {
  cuda_check({&d_out, &x});
  const int64_t n = x.size(-1);
  Tensor d_x = at::empty(x.sizes(), x.options());
  if (x.numel()) {
    const Tensor go = rows(d_out), xr = rows(x), dxr = d_x.view({-1, n});
    c10::cuda::CUDAGuard guard(x.device());
    check(fat_softmax_bwd(go.data_ptr(), xr.data_ptr(), dxr.data_ptr(), xr.size(0), n, go.stride(0), xr.stride(0), dxr.stride(0), eps,
                          dtype_tag(x), stream_of(x)));
  }
  return d_x;
}

// ------------------------------------------------------------------------------------- rational attention
Tensor unit_d(const Tensor& t) { return t.stride(-1) == 1 ? t : t.contiguous(); }

// [B,H,T,D] view whose memory order is (B,T,H,D), e.g. a slice of a packed QKV projection
bool is_token_major(const Tensor& t) { return t.dim() == 4 && t.size(1) > 1 && t.size(2) > 1 && t.stride(1) < t.stride(2); }

Tensor alloc_bhtd(const Tensor& like, bool token_major) {
  const int64_t B = like.size(0), H = like.size(1), T = like.size(2), D = like.size(3);
  if (token_major) return at::empty({B, T, H, D}, like.options()).permute({0, 2, 1, 3});
  return at::empty({B, H, T, D}, like.options());
}

// The packed padding mask of a launch (see fat_pack_key_mask), or null when there is none.
const uint32_t* mask_bits(const c10::optional<Tensor>& key_mask, const Tensor& q) {
  if (!key_mask.has_value() || !key_mask->defined()) return nullptr;
  const Tensor& m = *key_mask;
  TORCH_CHECK(m.is_cuda() && m.device() == q.device() && m.scalar_type() == at::kInt && m.is_contiguous() && m.dim() == 2 &&
              m.size(0) == q.size(0) && m.size(1) == fat_key_mask_words(int(q.size(2))),
              "key_mask must be the int32 [B, 4*ceil(T/128)] tensor that algebraic::pack_key_mask returns for these shapes");
  return reinterpret_cast<const uint32_t*>(m.data_ptr<int>());
}

// [B, T] mask (non-zero = the key takes part) -> int32 [B, 4*ceil(T/128)] bits for the attention operators.
Tensor pack_key_mask(const Tensor& mask) {
  cuda_check({&mask});
  TORCH_CHECK(mask.dim() == 2, "attention mask must be [B, T]");
  const Tensor m = mask.scalar_type() == at::kBool ? mask : mask.ne(0);
  const int64_t B = m.size(0), T = m.size(1);
  Tensor bits = at::empty({B, int64_t(fat_key_mask_words(int(T)))}, m.options().dtype(at::kInt));
  if (bits.numel()) {
    c10::cuda::CUDAGuard guard(m.device());
    check(fat_pack_key_mask(reinterpret_cast<const uint8_t*>(m.data_ptr<bool>()), reinterpret_cast<uint32_t*>(bits.data_ptr<int>()), int(B), int(T),
                            m.stride(0), m.stride(1), stream_of(m)));
  }
  return bits;
}

std::tuple<Tensor, Tensor, Tensor> attn_fwd(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, const Tensor& slopes, double scale,
                                            bool causal, double eps, int64_t path, bool token_major_out,
                                            const c10::optional<Tensor>& key_mask, bool residual) {
  cuda_check({&q_in, &k_in, &v_in, &slopes});
  TORCH_CHECK(q_in.dim() == 4 && q_in.sizes() == k_in.sizes() && q_in.sizes() == v_in.sizes() &&
              q_in.scalar_type() == k_in.scalar_type() && q_in.scalar_type() == v_in.scalar_type(), "q, k, v must be [B,H,T,D] of one shape and dtype");
  const Tensor q = unit_d(q_in), k = unit_d(k_in), v = unit_d(v_in);
  const int64_t B = q.size(0), H = q.size(1), T = q.size(2), D = q.size(3);
  const Tensor sl = slopes.to(at::kFloat).contiguous();
  TORCH_CHECK(sl.numel() == H, "alibi_slopes must hold one slope per head");
  Tensor out = alloc_bhtd(q, token_major_out);
  // 16-bit outputs also keep their rounding residual, so the backward can form Delta = dO.O accurately (`residual` false: the
  // caller knows no backward will follow and saves the second store pass, 5 % of the forward, and the tensor)
  Tensor out_lo = (q.element_size() == 2 && residual) ? alloc_bhtd(q, token_major_out) : at::empty({0}, q.options());
  Tensor L = at::empty({B, H, T}, q.options().dtype(at::kFloat));
  if (q.numel()) {
    c10::cuda::CUDAGuard guard(q.device());
    const auto qs = strides3(q), ks = strides3(k), vs = strides3(v), os = strides3(out);
    check(fat_attn_fwd_masked(q.data_ptr(), k.data_ptr(), v.data_ptr(), sl.data_ptr<float>(), mask_bits(key_mask, q), out.data_ptr(),
                       out_lo.numel() ? out_lo.data_ptr() : nullptr, L.data_ptr<float>(), int(B), int(H), int(T), int(D), qs.data(), ks.data(),
                       vs.data(), os.data(), scale, eps, int(causal), dtype_tag(q), int(path),
                       status_word(q.get_device()).data_ptr<int>(), stream_of(q)));
  }
  return {out, L, out_lo};
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, const Tensor& out_in,
                                            const Tensor& out_lo_in, const Tensor& L, const Tensor& d_out_in, const Tensor& slopes,
                                            double scale, bool causal, double eps, int64_t path, const c10::optional<Tensor>& key_mask) {
  cuda_check({&q_in, &k_in, &v_in, &out_in, &L, &d_out_in, &slopes});
  const Tensor q = unit_d(q_in), k = unit_d(k_in), v = unit_d(v_in), d_out = unit_d(d_out_in);
  Tensor out = unit_d(out_in), out_lo = out_lo_in;
  const int64_t B = q.size(0), H = q.size(1), T = q.size(2), D = q.size(3);
  void* lo_ptr = nullptr;
  if (out_lo.numel()) {
    if (out_lo.strides() != out.strides()) {       // the kernels address both with one set of strides
      out = out.contiguous();
      out_lo = out_lo.contiguous();
    }
    lo_ptr = out_lo.data_ptr();
  }
  const Tensor sl = slopes.to(at::kFloat).contiguous();
  const Tensor Lc = L.contiguous();
  Tensor d_q, d_k, d_v;
  if (is_token_major(q)) {
    // gradients of the three slices of a packed projection go into one [B,T,3,H,D] buffer
    Tensor packed = at::empty({B, T, 3, H, D}, q.options());
    d_q = packed.select(2, 0).permute({0, 2, 1, 3});
    d_k = packed.select(2, 1).permute({0, 2, 1, 3});
    d_v = packed.select(2, 2).permute({0, 2, 1, 3});
  } else {
    d_q = at::empty({B, H, T, D}, q.options());
    d_k = at::empty({B, H, T, D}, q.options());
    d_v = at::empty({B, H, T, D}, q.options());
  }
  if (q.numel()) {
    const int tag = dtype_tag(q);
    c10::cuda::CUDAGuard guard(q.device());
    const size_t ws_bytes = fat_attn_bwd_workspace_bytes(int(B), int(H), int(T), int(D), tag, int(path));
    Tensor ws = at::empty({int64_t(ws_bytes)}, q.options().dtype(at::kByte));
    const auto qs = strides3(q), ks = strides3(k), vs = strides3(v), os = strides3(out), dos = strides3(d_out), dqs = strides3(d_q),
               dks = strides3(d_k), dvs = strides3(d_v);
    check(fat_attn_bwd_masked(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lo_ptr, Lc.data_ptr<float>(), d_out.data_ptr(),
                       sl.data_ptr<float>(), mask_bits(key_mask, q), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), ws.data_ptr(), ws_bytes, int(B), int(H), int(T),
                       int(D), qs.data(), ks.data(), vs.data(), os.data(), dos.data(), dqs.data(), dks.data(), dvs.data(), scale, eps,
                       int(causal), tag, int(path), status_word(q.get_device()).data_ptr<int>(), stream_of(q)));
  }
  return {d_q, d_k, d_v};
}

// One decode step over a key/value cache: appends (k_new, v_new) at row n_cached[b] of the caches and returns the
// attention of the new token over rows 0..n_cached[b].  q, k_new, v_new [B,H,D]; caches [B,H,capacity,D].
Tensor attn_decode(const Tensor& q_in, const Tensor& k_new_in, const Tensor& v_new_in, Tensor& k_cache, Tensor& v_cache,
                   const Tensor& n_cached, const Tensor& slopes, double scale, double eps) {
  cuda_check({&q_in, &k_new_in, &v_new_in, &k_cache, &v_cache, &n_cached, &slopes});
  TORCH_CHECK(q_in.dim() == 3 && q_in.sizes() == k_new_in.sizes() && q_in.sizes() == v_new_in.sizes(), "q, k_new, v_new must be [B,H,D] of one shape");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.sizes() == v_cache.sizes() && k_cache.size(0) == q_in.size(0) && k_cache.size(1) == q_in.size(1) &&
              k_cache.size(3) == q_in.size(2), "the caches must be [B,H,capacity,D]");
  TORCH_CHECK(q_in.scalar_type() == k_new_in.scalar_type() && q_in.scalar_type() == v_new_in.scalar_type() &&
              q_in.scalar_type() == k_cache.scalar_type() && q_in.scalar_type() == v_cache.scalar_type(), "q, the new rows and the caches must share one dtype");
  TORCH_CHECK(k_cache.stride(3) == 1 && v_cache.stride(3) == 1, "the caches need unit stride along the head dimension");
  TORCH_CHECK(n_cached.scalar_type() == at::kInt && n_cached.dim() == 1 && n_cached.size(0) == q_in.size(0) && n_cached.is_contiguous(),
              "n_cached must be a dense int32 tensor of one length per sequence");
  auto unit = [](const Tensor& t) { return t.stride(-1) == 1 ? t : t.contiguous(); };
  const Tensor q = unit(q_in), k_new = unit(k_new_in), v_new = unit(v_new_in);
  const int64_t B = q.size(0), H = q.size(1), D = q.size(2);
  const Tensor sl = slopes.to(at::kFloat).contiguous();
  TORCH_CHECK(sl.numel() == H, "alibi_slopes must hold one slope per head");
  Tensor out = at::empty({B, H, D}, q.options());
  if (q.numel()) {
    c10::cuda::CUDAGuard guard(q.device());
    const std::array<int64_t, 2> qs{q.stride(0), q.stride(1)}, kns{k_new.stride(0), k_new.stride(1)}, vns{v_new.stride(0), v_new.stride(1)},
        os{out.stride(0), out.stride(1)};
    const auto kcs = strides3(k_cache), vcs = strides3(v_cache);
    check(fat_attn_decode(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), n_cached.data_ptr<int>(),
                          sl.data_ptr<float>(), out.data_ptr(), int(B), int(H), int(k_cache.size(2)), int(D), qs.data(), kns.data(), vns.data(),
                          os.data(), kcs.data(), vcs.data(), scale, eps, dtype_tag(q), status_word(q.get_device()).data_ptr<int>(), stream_of(q)));
  }
  return out;
}

}  // namespace

TORCH_LIBRARY(algebraic, m) {
  m.def("swiglu_fwd(Tensor gate, Tensor value) -> Tensor");
  m.def("swiglu_bwd(Tensor d_out, Tensor gate, Tensor value) -> (Tensor, Tensor)");
  m.def("norm_fwd(Tensor x, Tensor weight, float eps) -> (Tensor, Tensor)");
  m.def("norm_bwd(Tensor d_out, Tensor x, Tensor weight, Tensor mean, float eps) -> (Tensor, Tensor)");
  m.def("shifted_ce_fwd(Tensor logits, Tensor labels, int ignore_index) -> (Tensor, Tensor)");
  m.def("head_shifted_ce(Tensor y, Tensor weight, Tensor labels, int ignore_index, bool want_grads) -> (Tensor, Tensor, Tensor)");
  m.def("scale_unless_one(Tensor(a!) x, Tensor scale) -> ()");
  m.def("add_norm_fwd(Tensor x, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor, Tensor)");
  m.def("add_norm_bwd(Tensor d_y, Tensor? d_h, Tensor h, Tensor weight, Tensor mean, float eps) -> (Tensor, Tensor)");
  m.def("softmax_fwd(Tensor x, float eps) -> Tensor");
  m.def("softmax_bwd(Tensor d_out, Tensor x, float eps) -> Tensor");
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor slopes, float scale, bool causal, float eps, int path, "
        "bool token_major_out, Tensor? key_mask=None, bool residual=True) -> (Tensor, Tensor, Tensor)");
  m.def("attn_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor out_lo, Tensor L, Tensor d_out, Tensor slopes, "
        "float scale, bool causal, float eps, int path, Tensor? key_mask=None) -> (Tensor, Tensor, Tensor)");
  m.def("pack_key_mask(Tensor mask) -> Tensor");
  m.def("attn_decode(Tensor q, Tensor k_new, Tensor v_new, Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor n_cached, Tensor slopes, "
        "float scale, float eps) -> Tensor");
  m.def("device_status(int device) -> Tensor", &device_status);
}

TORCH_LIBRARY_IMPL(algebraic, CUDA, m) {
  m.impl("swiglu_fwd", &swiglu_fwd);
  m.impl("swiglu_bwd", &swiglu_bwd);
  m.impl("norm_fwd", &norm_fwd);
  m.impl("norm_bwd", &norm_bwd);
  m.impl("shifted_ce_fwd", &shifted_ce_fwd);
  m.impl("head_shifted_ce", &head_shifted_ce);
  m.impl("scale_unless_one", &scale_unless_one);
  m.impl("add_norm_fwd", &add_norm_fwd);
  m.impl("add_norm_bwd", &add_norm_bwd);
  m.impl("softmax_fwd", &softmax_fwd);
  m.impl("softmax_bwd", &softmax_bwd);
  m.impl("attn_fwd", &attn_fwd);
  m.impl("attn_bwd", &attn_bwd);
  m.impl("attn_decode", &attn_decode);
  m.impl("pack_key_mask", &pack_key_mask);
}
