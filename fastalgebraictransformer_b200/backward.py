"""Attention backward and the autograd entry point.

Host-side mirror of the reference's ``backward.py`` (rational_attention_backward 273-341,
RationalAttentionFunction 348-383, rational_attention 386-396).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib, ops  # noqa: F401
from .forward import compute_alibi_slopes, rational_attention_forward  # noqa: F401
from .fused_ops import EPS, NEG_INF  # noqa: F401


def rational_attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, output: torch.Tensor,
                                L: torch.Tensor, grad_output: torch.Tensor, alibi_slopes: torch.Tensor,
                                scale: float, causal: bool = True, eps: float = EPS,
                                path: int = _lib.PATH_AUTO,
                                output_lo: torch.Tensor = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward pass of rational attention (reference backward.py:273-341): returns (grad_q, grad_k, grad_v).

    ``output_lo`` is the optional rounding residual of a 16-bit ``output`` (what
    ``torch.ops.algebraic.attn_fwd`` returns third); without it Delta = dO.O is formed from the rounded output."""
    assert q.is_cuda
    lo = output_lo if output_lo is not None else q.new_empty(0)
    return torch.ops.algebraic.attn_bwd(q, k, v, output, lo, L, grad_output, alibi_slopes, float(scale), bool(causal),
                                        float(eps), int(path))


class RationalAttentionFunction(torch.autograd.Function):
    """Autograd function for rational attention (reference backward.py:348-383).

    ``apply(q, k, v, alibi_slopes, scale, causal, eps)``; the backward returns gradients for q, k, v only.
    """

    @staticmethod
    def forward(ctx, q, k, v, alibi_slopes, scale, causal, eps, path=_lib.PATH_AUTO, token_major_out=False):
        assert q.is_cuda and k.is_cuda and v.is_cuda
        assert q.shape == k.shape == v.shape
        output, L, output_lo = torch.ops.algebraic.attn_fwd(q, k, v, alibi_slopes, float(scale), bool(causal),
                                                            float(eps), int(path), bool(token_major_out))
        ctx.save_for_backward(q, k, v, output, L, output_lo, alibi_slopes)
        ctx.scale, ctx.causal, ctx.eps, ctx.path = float(scale), bool(causal), float(eps), int(path)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, output, L, output_lo, alibi_slopes = ctx.saved_tensors
        grad_q, grad_k, grad_v = torch.ops.algebraic.attn_bwd(q, k, v, output, output_lo, L, grad_output, alibi_slopes,
                                                              ctx.scale, ctx.causal, ctx.eps, ctx.path)
        return grad_q, grad_k, grad_v, None, None, None, None, None, None


def rational_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alibi_slopes: torch.Tensor, scale: float,
                       causal: bool = True, eps: float = EPS) -> torch.Tensor:
    """Memory-efficient rational attention with a custom backward (reference backward.py:386-396)."""
    if not q.is_cuda:
        raise RuntimeError("rational_attention: CUDA tensors required — this build has no CPU fallback")
    return RationalAttentionFunction.apply(q, k, v, alibi_slopes, scale, causal, eps)
