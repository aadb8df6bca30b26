"""``torch.library`` operators of the ``algebraic`` namespace.

The operators are defined and implemented in C++ (``csrc/torch_ops.cpp`` -> ``libfat_torch_ops.so``): each one
allocates its outputs with ATen, passes raw pointers / strides / the current CUDA stream to the C ABI of
``libfat_b200.so`` and turns a non-zero return code into ``RuntimeError``.  This module loads that library and
registers, from Python, the shape functions for meta tensors and the autograd formulas, so the operators compose with
``torch.utils.checkpoint`` (non-reentrant), DDP hooks and ``torch.autograd.grad``.  There is no Python or CPU
implementation behind them: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

_NS = "algebraic"
OPS_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libfat_torch_ops.so")


def _load() -> None:
    if hasattr(torch.ops.algebraic, "attn_fwd"):
        return
    for path in (_lib.LIB_PATH, OPS_LIB_PATH):
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `python -m fastalgebraictransformer_b200.build` "
                               "(nvcc for sm_100a, g++ for the operator registration).  This package has no fallback implementation.")
    _lib.lib()                                  # libfat_b200.so first: the operator library links against it
    torch.ops.load_library(OPS_LIB_PATH)


_load()
_alg = torch.ops.algebraic


def swiglu_bwd_packed(d_out: Tensor, gate: Tensor, value: Tensor) -> Tensor:
    """Both SwiGLU gradients as one [..., 2n] tensor (gate half first): what the gradient of the packed
    projection output needs, without a concatenation."""
    d_gate, _ = _alg.swiglu_bwd(d_out, gate, value)
    return d_gate._base if d_gate._base is not None else torch.cat(_alg.swiglu_bwd(d_out, gate, value), -1)


def head_shifted_ce(y: Tensor, weight: Tensor, labels: Tensor, ignore_index: int,
                    want_grads: bool = True) -> Tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """Loss head without the [B, T, V] logits: (loss, d_y, d_weight) of the mean cross-entropy between
    (y @ weight^T)[:, :-1] and labels[:, 1:] (reference algebraic_model.py:225-235).  The logits exist one sequence at a
    time.  With ``want_grads=False`` only the loss is computed and the two gradients are None."""
    loss, d_y, d_w = _alg.head_shifted_ce(y, weight, labels, int(ignore_index), bool(want_grads))
    return (loss, d_y, d_w) if want_grads else (loss, None, None)


def pack_key_mask(mask: Tensor) -> Tensor:
    """Padding mask [B, T] (non-zero = the key takes part; the reference's ``attention_mask``, algebraic_model.py:128-131)
    as the int32 [B, 4*ceil(T/128)] bit tensor the attention operators take; see include/fat_b200.h, fat_pack_key_mask."""
    return _alg.pack_key_mask(mask)


class PackedKeyMask:
    """A padding mask that has already been packed to bits (``bits``: int32 [B, 4*ceil(T/128)]), so that the layers of a
    model pack it once per step instead of once each."""

    def __init__(self, mask: Tensor):
        if mask.dim() != 2:
            raise ValueError("a padding mask must be [B, T]")
        self.n_tokens = mask.shape[1]
        self.bits = pack_key_mask(mask)


def as_key_mask_bits(key_mask, n_tokens: int) -> Optional[Tensor]:
    """None, a [B, T] padding mask (0 = padding) or a PackedKeyMask -> the bit tensor the attention operators take."""
    if key_mask is None:
        return None
    if not isinstance(key_mask, PackedKeyMask):
        key_mask = PackedKeyMask(key_mask)
    if key_mask.n_tokens != n_tokens:
        raise ValueError(f"the padding mask covers {key_mask.n_tokens} tokens, the sequence has {n_tokens}")
    return key_mask.bits


def attn_fwd(q: Tensor, k: Tensor, v: Tensor, slopes: Tensor, scale: float, causal: bool, eps: float,
             path: int, token_major_out: bool, key_mask: Optional[Tensor] = None, residual: bool = True) -> Tuple[Tensor, Tensor, Tensor]:
    """(out, L, out_lo) of rational attention; see include/fat_b200.h, fat_attn_fwd.  ``key_mask``: packed bits or None.
    ``residual=False``: no backward will follow, so the rounding residual of a 16-bit output is not written (out_lo is empty)."""
    return _alg.attn_fwd(q, k, v, slopes, float(scale), bool(causal), float(eps), int(path), bool(token_major_out), key_mask,
                         bool(residual))


def attn_decode(q: Tensor, k_new: Tensor, v_new: Tensor, k_cache: Tensor, v_cache: Tensor, n_cached: Tensor, slopes: Tensor,
                scale: float, eps: float) -> Tensor:
    """One decode step: appends the new key/value rows [B,H,D] at row n_cached[b] of the caches [B,H,capacity,D] and
    returns the new token's attention [B,H,D] over rows 0..n_cached[b]; see include/fat_b200.h, fat_attn_decode."""
    return _alg.attn_decode(q, k_new, v_new, k_cache, v_cache, n_cached, slopes, float(scale), float(eps))


def attn_bwd_packed(qkv: Tensor, out: Tensor, out_lo: Tensor, L: Tensor, d_out: Tensor, slopes: Tensor,
                    scale: float, causal: bool, eps: float, path: int, key_mask: Optional[Tensor] = None) -> Tensor:
    """Gradient of a packed [B,T,3,H,D] projection: d_q, d_k, d_v written side by side into one buffer."""
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    d_q, d_k, d_v = _alg.attn_bwd(q, k, v, out, out_lo, L, d_out, slopes, float(scale), bool(causal), float(eps), int(path), key_mask)
    base = d_q._base
    while base is not None and base._base is not None:
        base = base._base
    if base is None or base.shape != qkv.shape:           # q was not token-major after all (H == 1 or T == 1)
        base = torch.stack((d_q, d_k, d_v), 0).permute(1, 3, 0, 2, 4).contiguous()
    return base


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


@torch.library.register_fake(f"{_NS}::head_shifted_ce")
def _(y, weight, labels, ignore_index, want_grads):
    return (y.new_empty((), dtype=torch.float32), torch.empty_like(y) if want_grads else y.new_empty(0),
            torch.empty_like(weight) if want_grads else y.new_empty(0))


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


@torch.library.register_fake(f"{_NS}::pack_key_mask")
def _(mask):
    return mask.new_empty((mask.shape[0], 4 * ((mask.shape[1] + 127) // 128)), dtype=torch.int32)


@torch.library.register_fake(f"{_NS}::attn_fwd")
def _(q, k, v, slopes, scale, causal, eps, path, token_major_out, key_mask=None, residual=True):
    B, H, T, D = q.shape
    out = q.new_empty((B, T, H, D)).permute(0, 2, 1, 3) if token_major_out else q.new_empty((B, H, T, D))
    lo = torch.empty_like(out) if q.element_size() == 2 and residual else q.new_empty(0)
    return out, q.new_empty((B, H, T), dtype=torch.float32), lo


@torch.library.register_fake(f"{_NS}::attn_bwd")
def _(q, k, v, out, out_lo, L, d_out, slopes, scale, causal, eps, path, key_mask=None):
    return tuple(q.new_empty(q.shape) for _ in range(3))


@torch.library.register_fake(f"{_NS}::attn_decode")
def _(q, k_new, v_new, k_cache, v_cache, n_cached, slopes, scale, eps):
    return q.new_empty(q.shape)


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
    q, k, v, slopes, scale, causal, eps, path, _, key_mask, _residual = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1], output[2], slopes)
    ctx.args = (scale, causal, eps, path)
    ctx.key_mask = key_mask                                  # (an int32 tensor: nothing to differentiate)


def _attn_backward(ctx, d_out, d_L, d_lo):
    q, k, v, out, L, out_lo, slopes = ctx.saved_tensors
    d_q, d_k, d_v = torch.ops.algebraic.attn_bwd(q, k, v, out, out_lo, L, d_out, slopes, *ctx.args, ctx.key_mask)
    return d_q, d_k, d_v, None, None, None, None, None, None, None, None


torch.library.register_autograd(f"{_NS}::swiglu_fwd", _swiglu_backward, setup_context=_swiglu_setup)
torch.library.register_autograd(f"{_NS}::norm_fwd", _norm_backward, setup_context=_norm_setup)
torch.library.register_autograd(f"{_NS}::add_norm_fwd", _add_norm_backward, setup_context=_add_norm_setup)
torch.library.register_autograd(f"{_NS}::softmax_fwd", _softmax_backward, setup_context=_softmax_setup)
torch.library.register_autograd(f"{_NS}::attn_fwd", _attn_backward, setup_context=_attn_setup)
