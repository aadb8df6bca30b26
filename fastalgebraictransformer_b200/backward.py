"""Attention backward and the autograd entry point.

Host-side mirror of the reference's ``backward.py`` (rational_attention_backward 273-341,
RationalAttentionFunction 348-383, rational_attention 386-396).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops  # noqa: F401
from .ops import as_key_mask_bits
from .forward import compute_alibi_slopes, rational_attention_forward  # noqa: F401
from .fused_ops import EPS, NEG_INF  # noqa: F401


def rational_attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, output: torch.Tensor,
                                L: torch.Tensor, grad_output: torch.Tensor, alibi_slopes: torch.Tensor,
                                scale: float, causal: bool = True, eps: float = EPS,
                                path: int = _lib.PATH_AUTO, output_lo: torch.Tensor = None,
                                key_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward pass of rational attention (reference backward.py:273-341): returns (grad_q, grad_k, grad_v).

    ``output_lo`` is the optional rounding residual of a 16-bit ``output`` (what
    ``torch.ops.algebraic.attn_fwd`` returns third); without it Delta = dO.O is formed from the rounded output.
    ``key_mask``: the padding mask the forward was given, if any."""
    assert q.is_cuda
    lo = output_lo if output_lo is not None else q.new_empty(0)
    return torch.ops.algebraic.attn_bwd(q, k, v, output, lo, L, grad_output, alibi_slopes, float(scale), bool(causal),
                                        float(eps), int(path), as_key_mask_bits(key_mask, q.shape[2]))


class RationalAttentionFunction(torch.autograd.Function):
    """Autograd function for rational attention (reference backward.py:348-383).

    ``apply(q, k, v, alibi_slopes, scale, causal, eps)``; the backward returns gradients for q, k, v only.
    Extensions (optional trailing arguments): the kernel family, the memory order of the output, and ``key_mask``, a
    padding mask over the keys: [B, T] with 0 = padding as the reference's model takes it (algebraic_model.py:128-131),
    or an ``ops.PackedKeyMask`` made of one.
    """

    @staticmethod
    def forward(ctx, q, k, v, alibi_slopes, scale, causal, eps, path=_lib.PATH_AUTO, token_major_out=False, key_mask=None):
        assert q.is_cuda and k.is_cuda and v.is_cuda
        assert q.shape == k.shape == v.shape
        bits = as_key_mask_bits(key_mask, q.shape[2])
        output, L, output_lo = torch.ops.algebraic.attn_fwd(q, k, v, alibi_slopes, float(scale), bool(causal),
                                                            float(eps), int(path), bool(token_major_out), bits,
                                                            any(ctx.needs_input_grad[:3]))
        ctx.save_for_backward(q, k, v, output, L, output_lo, alibi_slopes)
        ctx.scale, ctx.causal, ctx.eps, ctx.path, ctx.bits = float(scale), bool(causal), float(eps), int(path), bits
        return output

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, output, L, output_lo, alibi_slopes = ctx.saved_tensors
        grad_q, grad_k, grad_v = torch.ops.algebraic.attn_bwd(q, k, v, output, output_lo, L, grad_output, alibi_slopes,
                                                              ctx.scale, ctx.causal, ctx.eps, ctx.path, ctx.bits)
        return grad_q, grad_k, grad_v, None, None, None, None, None, None, None


class RationalAttentionPackedFunction(torch.autograd.Function):
    """Causal rational attention straight from a packed projection ``qkv`` [B, T, 3, H, D] to [B, T, H*D].

    Same arithmetic as ``RationalAttentionFunction`` on the three permuted views (reference
    algebraic_model.py:89-107), but nothing is copied on either side: the kernels read the views in place,
    write the output in [B, T, H, D] order, and the backward returns one [B, T, 3, H, D] gradient."""

    @staticmethod
    def forward(ctx, qkv, alibi_slopes, scale, eps, key_mask=None):
        assert qkv.is_cuda and qkv.dim() == 5 and qkv.shape[2] == 3
        B, T, _, H, D = qkv.shape
        q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
        bits = as_key_mask_bits(key_mask, T)
        out, L, out_lo = ops.attn_fwd(q, k, v, alibi_slopes, float(scale), True, float(eps), _lib.PATH_AUTO, True, bits,
                                      ctx.needs_input_grad[0])
        ctx.save_for_backward(qkv, out, L, out_lo, alibi_slopes)
        ctx.scale, ctx.eps, ctx.bits = float(scale), float(eps), bits
        return out.permute(0, 2, 1, 3).reshape(B, T, H * D)        # a view: the memory order already is [B,T,H,D]

    @staticmethod
    def backward(ctx, grad_output):
        qkv, out, L, out_lo, alibi_slopes = ctx.saved_tensors
        B, T, _, H, D = qkv.shape
        d_out = grad_output.reshape(B, T, H, D).permute(0, 2, 1, 3)
        return ops.attn_bwd_packed(qkv, out, out_lo, L, d_out, alibi_slopes, ctx.scale, True, ctx.eps,
                                   _lib.PATH_AUTO, ctx.bits), None, None, None, None


def rational_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alibi_slopes: torch.Tensor, scale: float,
                       causal: bool = True, eps: float = EPS, key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Memory-efficient rational attention with a custom backward (reference backward.py:386-396).  ``key_mask`` (an
    extension): padding mask [B, T], 0 = the key is padding and weighs nothing for any query."""
    if not q.is_cuda:
        raise RuntimeError("rational_attention: CUDA tensors required — this build has no CPU fallback")
    if key_mask is None:
        return RationalAttentionFunction.apply(q, k, v, alibi_slopes, scale, causal, eps)
    return RationalAttentionFunction.apply(q, k, v, alibi_slopes, scale, causal, eps, _lib.PATH_AUTO, False, key_mask)
