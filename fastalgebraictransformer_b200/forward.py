"""Attention forward: ALiBi slopes and the forward launcher.

Host-side mirror of the reference's ``forward.py`` (compute_alibi_slopes 21-42,
rational_attention_forward 267-319).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib, ops  # noqa: F401
from .fused_ops import EPS, NEG_INF  # noqa: F401


def compute_alibi_slopes(n_heads: int, device: torch.device = None) -> torch.Tensor:
    """ALiBi slopes: 2^(-8(i+1)/n) for a power-of-two head count n; otherwise the slopes of the
    largest power of two p <= n followed by every other slope of 2p (reference forward.py:21-42)."""
    def geometric(n, idx):
        return torch.pow(2.0 ** (-(2.0 ** -(math.log2(n) - 3))), torch.as_tensor(list(idx)))

    p = 2 ** math.floor(math.log2(n_heads))
    slopes = geometric(p, range(1, p + 1))
    if p != n_heads:
        slopes = torch.cat([slopes, geometric(2 * p, range(1, 1 + 2 * min(p, n_heads - p), 2))])
    if device is not None:
        slopes = slopes.to(device)
    return slopes.float()


def rational_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, alibi_slopes: torch.Tensor,
                               scale: float, causal: bool = True, eps: float = EPS,
                               path: int = _lib.PATH_AUTO,
                               key_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward pass of rational attention (reference forward.py:267-319).

    q, k, v: [B, H, T, D] (any strides with unit stride along D are consumed in place).
    Returns ``(output [B,H,T,D], L [B,H,T] float32)``; L is the row sum of sigma^4 without eps.
    ``causal=False`` attends to every key with bias -slope*|i-j| (the reference accepts the flag
    but its kernels are always causal; the non-causal result is this package's extension).
    ``key_mask`` (an extension): padding mask [B, T], 0 = the key is padding (the reference's model applies one on its
    PyTorch path only, algebraic_model.py:128-131).
    """
    assert q.is_cuda and k.is_cuda and v.is_cuda
    assert q.shape == k.shape == v.shape
    out, L, _ = torch.ops.algebraic.attn_fwd(q.detach(), k.detach(), v.detach(), alibi_slopes, float(scale),
                                             bool(causal), float(eps), int(path), False,
                                             ops.as_key_mask_bits(key_mask, q.shape[2]), False)
    return out, L
