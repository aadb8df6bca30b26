"""``torch.library`` operators of the ``algebraic`` namespace, implemented by the C ABI.

Each operator allocates its outputs with torch, passes raw pointers / strides / the current
CUDA stream to libfat_b200.so and turns a non-zero return code into ``RuntimeError``.
Autograd formulas are registered on the forward operators, so they compose with
``torch.utils.checkpoint`` (non-reentrant), DDP hooks and ``torch.autograd.grad``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

_NS = "algebraic"
_libdef = torch.library.Library(_NS, "DEF")
_libdef.define("swiglu_fwd(Tensor gate, Tensor value) -> Tensor")
_libdef.define("swiglu_bwd(Tensor d_out, Tensor gate, Tensor value) -> (Tensor, Tensor)")
_libdef.define("norm_fwd(Tensor x, Tensor weight, float eps) -> (Tensor, Tensor)")
_libdef.define("norm_bwd(Tensor d_out, Tensor x, Tensor weight, Tensor mean, float eps) -> (Tensor, Tensor)")
_libdef.define("shifted_ce_fwd(Tensor logits, Tensor labels, int ignore_index) -> (Tensor, Tensor)")
_libdef.define("scale_unless_one(Tensor(a!) x, Tensor scale) -> ()")
_libdef.define("add_norm_fwd(Tensor x, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor, Tensor)")
_libdef.define("add_norm_bwd(Tensor d_y, Tensor? d_h, Tensor h, Tensor weight, Tensor mean, float eps) -> (Tensor, Tensor)")
_libdef.define("softmax_fwd(Tensor x, float eps) -> Tensor")
_libdef.define("softmax_bwd(Tensor d_out, Tensor x, float eps) -> Tensor")
_libdef.define("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor slopes, float scale, bool causal, float eps, "
               "int path, bool token_major_out) -> (Tensor, Tensor, Tensor)")
_libdef.define("attn_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor out_lo, Tensor L, Tensor d_out, Tensor slopes, "
               "float scale, bool causal, float eps, int path) -> (Tensor, Tensor, Tensor)")


def _p(t: Tensor) -> int:
    return t.data_ptr()


def _rows(t: Tensor) -> Tensor:
    """View ``t`` as [n_rows, n_cols] with unit column stride, copying only when it must."""
    n = t.shape[-1]
    if t.dim() == 2 and t.stride(1) == 1:
        return t
    if t.stride(-1) == 1 or n == 1:
        try:
            return t.view(-1, n)           # fails for views that cannot be flattened
        except RuntimeError:
            pass
        # a slice of the last dimension of a dense tensor (e.g. one half of chunk(2,-1)): rows are
        # equally spaced, so (n_rows, row_stride) describes it without a copy
        st = t.stride(-2) if t.dim() >= 2 else n
        ok, expect = True, st
        for d in range(t.dim() - 2, -1, -1):
            if t.shape[d] != 1 and t.stride(d) != expect:
                ok = False
                break
            expect = t.stride(d) * t.shape[d]
        if ok:
            return t.as_strided((t.numel() // n, n), (st, 1), t.storage_offset())
    return t.contiguous().view(-1, n)


def _cuda_check(*ts: Tensor) -> None:
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("algebraic ops run on CUDA tensors only (there is no CPU fallback)")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")


# ----------------------------------------------------------------------------- SwiGLU
def _swiglu_fwd(gate: Tensor, value: Tensor) -> Tensor:
    _cuda_check(gate, value)
    assert gate.shape == value.shape and gate.dtype == value.dtype
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    if gate.numel() == 0:
        return out
    g, v, o = _rows(gate), _rows(value), out.view(-1, gate.shape[-1])
    with _lib.device_guard(gate.device):
        _lib.check(_lib.lib().fat_swiglu_fwd(_p(g), _p(v), _p(o), g.shape[0], g.shape[1], g.stride(0), v.stride(0),
                                             o.stride(0), _lib.dtype_tag(gate), _lib.stream_ptr(gate.device)))
    return out


def _swiglu_bwd(d_out: Tensor, gate: Tensor, value: Tensor) -> Tuple[Tensor, Tensor]:
    _cuda_check(d_out, gate, value)
    n = gate.shape[-1]
    # both gradients live in one [rows, 2n] buffer: when gate/value were the two halves of a packed
    # projection, autograd's concatenation of the halves becomes a no-op copy target of the same layout
    packed = torch.empty(gate.shape[:-1] + (2 * n,), dtype=gate.dtype, device=gate.device)
    d_gate, d_value = packed[..., :n], packed[..., n:]
    if gate.numel() == 0:
        return d_gate, d_value
    go, g, v = _rows(d_out), _rows(gate), _rows(value)
    dg, dv = _rows(d_gate), _rows(d_value)
    with _lib.device_guard(gate.device):
        _lib.check(_lib.lib().fat_swiglu_bwd(_p(go), _p(g), _p(v), _p(dg), _p(dv), g.shape[0], n, go.stride(0),
                                             g.stride(0), v.stride(0), dg.stride(0), dv.stride(0),
                                             _lib.dtype_tag(gate), _lib.stream_ptr(gate.device)))
    return d_gate, d_value


def swiglu_bwd_packed(d_out: Tensor, gate: Tensor, value: Tensor) -> Tensor:
    """Both SwiGLU gradients as one [..., 2n] tensor (gate half first): what the gradient of the packed
    projection output needs, without a concatenation."""
    d_gate, _ = _swiglu_bwd(d_out, gate, value)
    return d_gate._base if d_gate._base is not None else torch.cat(_swiglu_bwd(d_out, gate, value), -1)


# ----------------------------------------------------------------------------- mean-error norm
def _norm_fwd(x: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    _cuda_check(x, weight)
    n = x.shape[-1]
    assert weight.shape == (n,), "weight must be [n_cols]"
    w = weight.to(x.dtype).contiguous()
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    xr = _rows(x)
    mean = torch.empty(xr.shape[0], dtype=torch.float32, device=x.device)
    if x.numel():
        yr = y.view(-1, n)
        with _lib.device_guard(x.device):
            _lib.check(_lib.lib().fat_norm_fwd(_p(xr), _p(w), _p(yr), _p(mean), xr.shape[0], n, xr.stride(0),
                                               yr.stride(0), eps, _lib.dtype_tag(x), _lib.stream_ptr(x.device)))
    return y, mean


def _norm_bwd(d_out: Tensor, x: Tensor, weight: Tensor, mean: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    _cuda_check(d_out, x, weight, mean)
    n = x.shape[-1]
    w = weight.to(x.dtype).contiguous()
    d_x = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    d_w = torch.empty(n, dtype=x.dtype, device=x.device)
    go, xr, dxr = _rows(d_out), _rows(x), d_x.view(-1, n)
    tag = _lib.dtype_tag(x)
    L = _lib.lib()
    ws_bytes = L.fat_norm_bwd_workspace_bytes(xr.shape[0], n, tag)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _lib.device_guard(x.device):
        _lib.check(L.fat_norm_bwd(_p(go), _p(xr), _p(w), _p(mean), _p(dxr), _p(d_w), _p(ws), ws_bytes, xr.shape[0], n,
                                  go.stride(0) if go.numel() else n, xr.stride(0) if xr.numel() else n, n,
                                  eps, tag, _lib.stream_ptr(x.device)))
    return d_x, d_w.to(weight.dtype)


def _add_norm_fwd(x: Tensor, residual: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor, Tensor]:
    """h = x + residual, y = mean_error_norm(h, weight), in one pass.  Returns (h, y, mean)."""
    _cuda_check(x, residual, weight)
    assert x.shape == residual.shape and x.dtype == residual.dtype, "x and residual must match"
    n = x.shape[-1]
    assert weight.shape == (n,), "weight must be [n_cols]"
    w = weight.to(x.dtype).contiguous()
    h = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    xr, rr = _rows(x), _rows(residual)
    mean = torch.empty(xr.shape[0], dtype=torch.float32, device=x.device)
    if x.numel():
        hr, yr = h.view(-1, n), y.view(-1, n)
        with _lib.device_guard(x.device):
            _lib.check(_lib.lib().fat_add_norm_fwd(_p(xr), _p(rr), _p(w), _p(hr), _p(yr), _p(mean), xr.shape[0], n,
                                                   xr.stride(0), rr.stride(0), n, n, eps, _lib.dtype_tag(x),
                                                   _lib.stream_ptr(x.device)))
    return h, y, mean


def _add_norm_bwd(d_y: Tensor, d_h: Optional[Tensor], h: Tensor, weight: Tensor, mean: Tensor,
                  eps: float) -> Tuple[Tensor, Tensor]:
    """Gradient of the sum (shared by x and residual) and of the weight."""
    _cuda_check(d_y, h, weight, mean)
    n = h.shape[-1]
    w = weight.to(h.dtype).contiguous()
    d_sum = torch.empty(h.shape, dtype=h.dtype, device=h.device)
    d_w = torch.empty(n, dtype=h.dtype, device=h.device)
    go, hr, dsr = _rows(d_y), _rows(h), d_sum.view(-1, n)
    dh = _rows(d_h.to(h.dtype)) if d_h is not None else None
    tag = _lib.dtype_tag(h)
    L = _lib.lib()
    ws_bytes = L.fat_norm_bwd_workspace_bytes(hr.shape[0], n, tag)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=h.device)
    with _lib.device_guard(h.device):
        _lib.check(L.fat_add_norm_bwd(_p(go), _p(dh) if dh is not None and dh.numel() else None, _p(hr), _p(w), _p(mean),
                                      _p(dsr), _p(d_w), _p(ws), ws_bytes, hr.shape[0], n,
                                      go.stride(0) if go.numel() else n, dh.stride(0) if dh is not None and dh.numel() else n,
                                      hr.stride(0) if hr.numel() else n, n, eps, tag, _lib.stream_ptr(h.device)))
    return d_sum, d_w.to(weight.dtype)


# ----------------------------------------------------------------------------- shifted cross-entropy (loss head)
def _shifted_ce_fwd(logits: Tensor, labels: Tensor, ignore_index: int) -> Tuple[Tensor, Tensor]:
    """(loss, d_logits) of mean cross-entropy between logits[:, :-1] and labels[:, 1:]; loss is a float32 scalar and
    d_logits ([B, T, V], dtype of logits) is its gradient with respect to logits."""
    _cuda_check(logits, labels)
    assert logits.dim() == 3 and labels.shape == logits.shape[:2] and labels.dtype == torch.int64
    if logits.stride(2) != 1:
        logits = logits.contiguous()
    B, T, V = logits.shape
    counted = labels[:, 1:]
    n_valid = ((counted != ignore_index) & (counted >= 0) & (counted < V)).sum().to(torch.float32).reshape(1)
    row_loss = torch.empty(B * T, dtype=torch.float32, device=logits.device)
    d_logits = torch.empty((B, T, V), dtype=logits.dtype, device=logits.device)
    if logits.numel():
        with _lib.device_guard(logits.device):
            _lib.check(_lib.lib().fat_shifted_ce_fwd(_p(logits), _p(labels), _p(n_valid), _p(row_loss), _p(d_logits), B, T, V,
                                                     logits.stride(0), logits.stride(1), labels.stride(0), labels.stride(1),
                                                     ignore_index, _lib.dtype_tag(logits), _lib.stream_ptr(logits.device)))
    loss = row_loss.sum() / n_valid.clamp_min(1.0).squeeze(0) if logits.numel() else row_loss.sum()
    return loss, d_logits


def head_shifted_ce(y: Tensor, weight: Tensor, labels: Tensor, ignore_index: int,
                    want_grads: bool = True) -> Tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """Loss head without the [B, T, V] logits: (loss, d_y, d_weight) of the mean cross-entropy between
    (y @ weight^T)[:, :-1] and labels[:, 1:] (reference algebraic_model.py:225-235).

    The logits exist one sequence at a time: a [T, V] buffer is filled by the head GEMM, the loss kernel turns it in
    place into its own gradient, and two more GEMMs fold that gradient into d_y [B, T, C] and d_weight [V, C] before the
    buffer is reused for the next sequence.  With ``want_grads=False`` only the loss is computed."""
    _cuda_check(y, weight, labels)
    assert y.dim() == 3 and weight.dim() == 2 and y.shape[2] == weight.shape[1] and labels.shape == y.shape[:2]
    assert labels.dtype == torch.int64 and y.dtype == weight.dtype
    B, T, C = y.shape
    V = weight.shape[0]
    y = y.contiguous()
    counted = labels[:, 1:]
    n_valid = ((counted != ignore_index) & (counted >= 0) & (counted < V)).sum().to(torch.float32).reshape(1)
    row_loss = torch.zeros(B * T, dtype=torch.float32, device=y.device)
    d_y = torch.empty_like(y) if want_grads else None
    d_w = torch.empty_like(weight) if want_grads else None
    if y.numel() and V:
        buf = torch.empty((T, V), dtype=y.dtype, device=y.device)
        lib, tag, wt = _lib.lib(), _lib.dtype_tag(y), weight.t()
        with _lib.device_guard(y.device):
            for b in range(B):
                torch.mm(y[b], wt, out=buf)
                _lib.check(lib.fat_shifted_ce_fwd(_p(buf), _p(labels[b]), _p(n_valid), _p(row_loss[b * T:]),
                                                  _p(buf) if want_grads else None, 1, T, V, T * V, V,
                                                  labels.stride(0), labels.stride(1), ignore_index, tag,
                                                  _lib.stream_ptr(y.device)))
                if want_grads:
                    torch.mm(buf, weight, out=d_y[b])
                    if b == 0:
                        torch.mm(buf.t(), y[b], out=d_w)
                    else:
                        d_w.addmm_(buf.t(), y[b])
    elif want_grads:
        d_w.zero_()
    loss = row_loss.sum() / n_valid.clamp_min(1.0).squeeze(0)
    return loss, d_y, d_w


def _scale_unless_one(x: Tensor, scale: Tensor) -> None:
    _cuda_check(x, scale)
    assert x.is_contiguous() and scale.dtype == torch.float32 and scale.numel() == 1
    if x.numel():
        with _lib.device_guard(x.device):
            _lib.check(_lib.lib().fat_scale_unless_one(_p(x), x.numel(), _p(scale), _lib.dtype_tag(x), _lib.stream_ptr(x.device)))


# ----------------------------------------------------------------------------- rational softmax
def _softmax_fwd(x: Tensor, eps: float) -> Tensor:
    _cuda_check(x)
    n = x.shape[-1]
    p = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if x.numel():
        xr, pr = _rows(x), p.view(-1, n)
        with _lib.device_guard(x.device):
            _lib.check(_lib.lib().fat_softmax_fwd(_p(xr), _p(pr), xr.shape[0], n, xr.stride(0), pr.stride(0), eps,
                                                  _lib.dtype_tag(x), _lib.stream_ptr(x.device)))
    return p


def _softmax_bwd(d_out: Tensor, x: Tensor, eps: float) -> Tensor:
    _cuda_check(d_out, x)
    n = x.shape[-1]
    d_x = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if x.numel():
        go, xr, dxr = _rows(d_out), _rows(x), d_x.view(-1, n)
        with _lib.device_guard(x.device):
            _lib.check(_lib.lib().fat_softmax_bwd(_p(go), _p(xr), _p(dxr), xr.shape[0], n, go.stride(0), xr.stride(0),
                                                  dxr.stride(0), eps, _lib.dtype_tag(x), _lib.stream_ptr(x.device)))
    return d_x


# ----------------------------------------------------------------------------- rational attention
def _unit_d(t: Tensor) -> Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _is_token_major(t: Tensor) -> bool:
    """[B,H,T,D] view whose memory order is (B,T,H,D), e.g. a slice of a packed QKV projection."""
    return t.dim() == 4 and t.shape[1] > 1 and t.shape[2] > 1 and t.stride(1) < t.stride(2)


def _alloc_bhtd(like: Tensor, token_major: bool) -> Tensor:
    B, H, T, D = like.shape
    if token_major:
        return torch.empty((B, T, H, D), dtype=like.dtype, device=like.device).permute(0, 2, 1, 3)
    return torch.empty((B, H, T, D), dtype=like.dtype, device=like.device)


def _attn_fwd(q: Tensor, k: Tensor, v: Tensor, slopes: Tensor, scale: float, causal: bool, eps: float,
              path: int, token_major_out: bool) -> Tuple[Tensor, Tensor, Tensor]:
    _cuda_check(q, k, v, slopes)
    assert q.dim() == 4 and q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype
    B, H, T, D = q.shape
    q, k, v = _unit_d(q), _unit_d(k), _unit_d(v)
    sl = slopes.to(torch.float32).contiguous()
    assert sl.numel() == H, "alibi_slopes must hold one slope per head"
    out = _alloc_bhtd(q, token_major_out)
    # 16-bit outputs also keep their rounding residual, so the backward can form Delta = dO.O accurately
    out_lo = _alloc_bhtd(q, token_major_out) if q.element_size() == 2 else q.new_empty(0)
    L = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    if q.numel():
        with _lib.device_guard(q.device):
            _lib.check(_lib.lib().fat_attn_fwd(
                _p(q), _p(k), _p(v), _p(sl), _p(out), _p(out_lo) if out_lo.numel() else None, _p(L), B, H, T, D,
                _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out),
                scale, eps, int(causal), _lib.dtype_tag(q), path,
                _p(_lib.device_status(q.device)), _lib.stream_ptr(q.device)))
    return out, L, out_lo


def _attn_bwd(q: Tensor, k: Tensor, v: Tensor, out: Tensor, out_lo: Tensor, L: Tensor, d_out: Tensor, slopes: Tensor,
              scale: float, causal: bool, eps: float, path: int) -> Tuple[Tensor, Tensor, Tensor]:
    _cuda_check(q, k, v, out, L, d_out, slopes)
    B, H, T, D = q.shape
    q, k, v, out, d_out = _unit_d(q), _unit_d(k), _unit_d(v), _unit_d(out), _unit_d(d_out)
    lo_ptr = None
    if out_lo.numel():
        if out_lo.stride() != out.stride():       # the kernels address both with one set of strides
            out, out_lo = out.contiguous(), out_lo.contiguous()
        lo_ptr = _p(out_lo)
    sl = slopes.to(torch.float32).contiguous()
    Lc = L.contiguous()
    if _is_token_major(q):
        # gradients of the three slices of a packed projection go into one [B,T,3,H,D] buffer
        packed = torch.empty((B, T, 3, H, D), dtype=q.dtype, device=q.device)
        d_q, d_k, d_v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    else:
        d_q, d_k, d_v = (torch.empty((B, H, T, D), dtype=q.dtype, device=q.device) for _ in range(3))
    if q.numel():
        lib = _lib.lib()
        tag = _lib.dtype_tag(q)
        ws_bytes = lib.fat_attn_bwd_workspace_bytes(B, H, T, D, tag, path)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        with _lib.device_guard(q.device):
            _lib.check(lib.fat_attn_bwd(
                _p(q), _p(k), _p(v), _p(out), lo_ptr, _p(Lc), _p(d_out), _p(sl), _p(d_q), _p(d_k), _p(d_v),
                _p(ws), ws_bytes, B, H, T, D,
                _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), _lib.strides3(d_out),
                _lib.strides3(d_q), _lib.strides3(d_k), _lib.strides3(d_v),
                scale, eps, int(causal), tag, path, _p(_lib.device_status(q.device)), _lib.stream_ptr(q.device)))
    return d_q, d_k, d_v


def attn_bwd_packed(qkv: Tensor, out: Tensor, out_lo: Tensor, L: Tensor, d_out: Tensor, slopes: Tensor,
                    scale: float, causal: bool, eps: float, path: int) -> Tensor:
    """Gradient of a packed [B,T,3,H,D] projection: d_q, d_k, d_v written side by side into one buffer."""
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    d_q, d_k, d_v = _attn_bwd(q, k, v, out, out_lo, L, d_out, slopes, scale, causal, eps, path)
    base = d_q._base
    if base is None or base.shape != qkv.shape:           # q was not token-major after all (H == 1 or T == 1)
        base = torch.stack((d_q, d_k, d_v), 0).permute(1, 3, 0, 2, 4).contiguous()
    return base


for _name, _fn in (("swiglu_fwd", _swiglu_fwd), ("swiglu_bwd", _swiglu_bwd), ("norm_fwd", _norm_fwd),
                   ("norm_bwd", _norm_bwd), ("add_norm_fwd", _add_norm_fwd), ("add_norm_bwd", _add_norm_bwd),
                   ("shifted_ce_fwd", _shifted_ce_fwd), ("scale_unless_one", _scale_unless_one),
                   ("softmax_fwd", _softmax_fwd), ("softmax_bwd", _softmax_bwd),
                   ("attn_fwd", _attn_fwd), ("attn_bwd", _attn_bwd)):
    _libdef.impl(_name, _fn, "CUDA")


# ----------------------------------------------------------------------------- shape functions (meta)
@torch.library.register_fake(f"{_NS}::swiglu_fwd")
def _(gate, value):
    return torch.empty_like(gate, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{_NS}::swiglu_bwd")
def _(d_out, gate, value):
    n = gate.shape[-1]
    packed = gate.new_empty(gate.shape[:-1] + (2 * n,))
    return packed[..., :n], packed[..., n:]


@torch.library.register_fake(f"{_NS}::norm_fwd")
def _(x, weight, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32)


@torch.library.register_fake(f"{_NS}::norm_bwd")
def _(d_out, x, weight, mean, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight)


@torch.library.register_fake(f"{_NS}::shifted_ce_fwd")
def _(logits, labels, ignore_index):
    return logits.new_empty((), dtype=torch.float32), torch.empty_like(logits, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{_NS}::scale_unless_one")
def _(x, scale):
    return None


@torch.library.register_fake(f"{_NS}::add_norm_fwd")
def _(x, residual, weight, eps):
    return (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(x, memory_format=torch.contiguous_format),
            x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32))


@torch.library.register_fake(f"{_NS}::add_norm_bwd")
def _(d_y, d_h, h, weight, mean, eps):
    return torch.empty_like(h, memory_format=torch.contiguous_format), torch.empty_like(weight)


@torch.library.register_fake(f"{_NS}::softmax_fwd")
def _(x, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{_NS}::softmax_bwd")
def _(d_out, x, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{_NS}::attn_fwd")
def _(q, k, v, slopes, scale, causal, eps, path, token_major_out):
    B, H, T, D = q.shape
    out = q.new_empty((B, T, H, D)).permute(0, 2, 1, 3) if token_major_out else q.new_empty((B, H, T, D))
    lo = torch.empty_like(out) if q.element_size() == 2 else q.new_empty(0)
    return out, q.new_empty((B, H, T), dtype=torch.float32), lo


@torch.library.register_fake(f"{_NS}::attn_bwd")
def _(q, k, v, out, out_lo, L, d_out, slopes, scale, causal, eps, path):
    return tuple(q.new_empty(q.shape) for _ in range(3))


# ----------------------------------------------------------------------------- autograd formulas
def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swiglu_backward(ctx, d_out):
    gate, value = ctx.saved_tensors
    return torch.ops.algebraic.swiglu_bwd(d_out, gate, value)


def _norm_setup(ctx, inputs, output):
    x, weight, eps = inputs
    ctx.save_for_backward(x, weight, output[1])
    ctx.eps = eps


def _norm_backward(ctx, d_y, d_mean):
    x, weight, mean = ctx.saved_tensors
    d_x, d_w = torch.ops.algebraic.norm_bwd(d_y, x, weight, mean, ctx.eps)
    return d_x, d_w, None


def _add_norm_setup(ctx, inputs, output):
    x, residual, weight, eps = inputs
    ctx.save_for_backward(output[0], weight, output[2])      # h, not x and residual: the backward only needs their sum
    ctx.eps = eps


def _add_norm_backward(ctx, d_h, d_y, d_mean):
    h, weight, mean = ctx.saved_tensors
    if d_y is None:                                          # only the sum was used downstream
        return d_h, d_h, None, None
    d_sum, d_w = torch.ops.algebraic.add_norm_bwd(d_y, d_h, h, weight, mean, ctx.eps)
    return d_sum, d_sum, d_w, None


def _softmax_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])
    ctx.eps = inputs[1]


def _softmax_backward(ctx, d_out):
    (x,) = ctx.saved_tensors
    return torch.ops.algebraic.softmax_bwd(d_out, x, ctx.eps), None


def _attn_setup(ctx, inputs, output):
    q, k, v, slopes, scale, causal, eps, path, _ = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1], output[2], slopes)
    ctx.args = (scale, causal, eps, path)


def _attn_backward(ctx, d_out, d_L, d_lo):
    q, k, v, out, L, out_lo, slopes = ctx.saved_tensors
    d_q, d_k, d_v = torch.ops.algebraic.attn_bwd(q, k, v, out, out_lo, L, d_out, slopes, *ctx.args)
    return d_q, d_k, d_v, None, None, None, None, None, None


torch.library.register_autograd(f"{_NS}::swiglu_fwd", _swiglu_backward, setup_context=_swiglu_setup)
torch.library.register_autograd(f"{_NS}::norm_fwd", _norm_backward, setup_context=_norm_setup)
torch.library.register_autograd(f"{_NS}::add_norm_fwd", _add_norm_backward, setup_context=_add_norm_setup)
torch.library.register_autograd(f"{_NS}::softmax_fwd", _softmax_backward, setup_context=_softmax_setup)
torch.library.register_autograd(f"{_NS}::attn_fwd", _attn_backward, setup_context=_attn_setup)
