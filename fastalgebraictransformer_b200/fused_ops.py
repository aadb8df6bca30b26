"""Fused element-wise / row operators: rational softmax, rational SwiGLU, mean-error norm.

Host-side mirror of the reference's ``fused_ops.py`` (autograd Functions 435-599 and the
convenience functions 606-636): same names, argument meaning and assertion behaviour.  The
work is done by the sm_100a kernels behind ``torch.ops.algebraic.*``; CPU tensors are
rejected (this package carries no fallback implementation).
"""
from __future__ import annotations

import torch

from . import ops  # noqa: F401  (registers torch.ops.algebraic)

EPS = 1e-6      # added to sums / means, never inside sigma (reference fused_ops.py:20)
NEG_INF = -1e4  # kept for API parity (reference fused_ops.py:21); the kernels skip masked keys instead

_alg = torch.ops.algebraic


class RationalSoftmax(torch.autograd.Function):
    """p = sigma(x)^4 / (sum sigma(x)^4 + eps) over the last dimension (reference fused_ops.py:435-487)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
        assert x.is_cuda, "Input must be on CUDA"
        out = _alg.softmax_fwd(x, eps)
        ctx.save_for_backward(x)
        ctx.eps = eps
        return out

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        (x,) = ctx.saved_tensors
        return _alg.softmax_bwd(grad_output, x, ctx.eps), None


class RationalSwiGLU(torch.autograd.Function):
    """out = gate * sigma(gate) * value (reference fused_ops.py:490-539)."""

    @staticmethod
    def forward(ctx, gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        assert gate.is_cuda and value.is_cuda, "Inputs must be on CUDA"
        out = _alg.swiglu_fwd(gate, value)
        ctx.save_for_backward(gate, value)
        return out

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        gate, value = ctx.saved_tensors
        return _alg.swiglu_bwd(grad_output, gate, value)


class RationalSwiGLUPacked(torch.autograd.Function):
    """Rational SwiGLU of a packed projection ``gv = [gate | value]`` (last dimension 2n -> n).

    What ``RationalSwiGLU.apply(*gv.chunk(2, -1))`` computes, but the backward hands autograd ONE
    [..., 2n] gradient instead of two halves that it would have to concatenate.  Used by the model's FFN
    (reference algebraic_model.py:51-62)."""

    @staticmethod
    def forward(ctx, gv: torch.Tensor) -> torch.Tensor:
        assert gv.is_cuda, "Inputs must be on CUDA"
        gate, value = gv.chunk(2, dim=-1)
        ctx.save_for_backward(gv)
        return _alg.swiglu_fwd(gate, value)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        (gv,) = ctx.saved_tensors
        gate, value = gv.chunk(2, dim=-1)
        return ops.swiglu_bwd_packed(grad_output, gate, value)


class MeanErrorNorm(torch.autograd.Function):
    """y = x / (mean|x| + eps) * weight (reference fused_ops.py:542-599); returns (d_x, d_weight, None)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor, eps: float = EPS) -> torch.Tensor:
        assert x.is_cuda, "Input must be on CUDA"
        y, mean = _alg.norm_fwd(x, weight, eps)
        ctx.save_for_backward(x, weight, mean)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        x, weight, mean = ctx.saved_tensors
        d_x, d_w = _alg.norm_bwd(grad_output, x, weight, mean, ctx.eps)
        return d_x, d_w, None


class AddMeanErrorNorm(torch.autograd.Function):
    """(h, y) with h = x + residual and y = mean_error_norm(h, weight): the residual addition of a pre-norm block fused
    with the normalisation that follows it (reference algebraic_model.py:149-152 does the two in separate passes).
    backward returns (d_sum, d_sum, d_weight, None) with d_sum = d_h + d(norm)/dh."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = EPS):
        assert x.is_cuda and residual.is_cuda, "Input must be on CUDA"
        h, y, mean = _alg.add_norm_fwd(x, residual, weight, eps)
        ctx.save_for_backward(h, weight, mean)
        ctx.eps = eps
        ctx.set_materialize_grads(False)             # an unused result arrives as None, not as a tensor of zeros
        return h, y

    @staticmethod
    def backward(ctx, d_h, d_y):
        h, weight, mean = ctx.saved_tensors
        if d_y is None:                              # only the sum was used downstream
            return d_h, d_h, None, None
        d_sum, d_w = _alg.add_norm_bwd(d_y, d_h, h, weight, mean, ctx.eps)
        return d_sum, d_sum, d_w, None


class ShiftedCrossEntropy(torch.autograd.Function):
    """Mean cross-entropy of logits[:, :-1] against labels[:, 1:] (reference algebraic_model.py:229-235) with the gradient
    produced by the same pass over the logits; the backward multiplies it by the incoming scalar (a no-op when it is 1)."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
        assert logits.is_cuda, "Input must be on CUDA"
        loss, d_logits = _alg.shifted_ce_fwd(logits, labels, ignore_index)
        ctx.save_for_backward(d_logits)
        return loss.to(logits.dtype)

    @staticmethod
    def backward(ctx, grad_loss):
        (d_logits,) = ctx.saved_tensors
        if getattr(ctx, "consumed", False):
            # the gradient is scaled in place to avoid a second [B, T, V] tensor; a second pass over the same graph
            # (retain_graph=True) would scale it twice
            raise RuntimeError("ShiftedCrossEntropy: backward through the same forward twice is not supported "
                               "(its saved gradient is scaled in place); run the forward again")
        ctx.consumed = True
        _alg.scale_unless_one(d_logits, grad_loss.to(torch.float32).reshape(1))
        return d_logits, None, None


class HeadShiftedCrossEntropy(torch.autograd.Function):
    """Loss of the language-model head, ``cross_entropy((y @ weight^T)[:, :-1], labels[:, 1:])`` (reference
    algebraic_model.py:225-235), for callers that do not keep the logits: the [B, T, V] tensor and its gradient never
    exist, only one sequence's [T, V] slice at a time.  The gradients with respect to ``y`` and ``weight`` are formed in
    the forward (they need the same slices) and scaled by the incoming scalar in the backward."""

    @staticmethod
    def forward(ctx, y: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
        assert y.is_cuda, "Input must be on CUDA"
        want = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        loss, d_y, d_w = ops.head_shifted_ce(y, weight, labels, ignore_index, want_grads=want)
        if want:
            ctx.save_for_backward(d_y, d_w)
        return loss.to(y.dtype)

    @staticmethod
    def backward(ctx, grad_loss):
        d_y, d_w = ctx.saved_tensors
        if getattr(ctx, "consumed", False):
            raise RuntimeError("HeadShiftedCrossEntropy: backward through the same forward twice is not supported "
                               "(its saved gradients are scaled in place); run the forward again")
        ctx.consumed = True
        scale = grad_loss.to(torch.float32).reshape(1)
        _alg.scale_unless_one(d_y, scale)
        _alg.scale_unless_one(d_w, scale)
        return d_y, d_w, None, None


def head_shifted_cross_entropy(y: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               ignore_index: int = -100) -> torch.Tensor:
    """Next-token loss of ``y @ weight^T`` against ``labels`` without materialising the logits."""
    _require_cuda(y, "head_shifted_cross_entropy")
    return HeadShiftedCrossEntropy.apply(y, weight, labels, ignore_index)


def shifted_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Next-token loss of a [B, T, V] logits tensor against [B, T] labels, as the model computes it."""
    _require_cuda(logits, "shifted_cross_entropy")
    return ShiftedCrossEntropy.apply(logits, labels, ignore_index)


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: CUDA tensor required — this build has no CPU fallback")


def rational_softmax(x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """Apply rational softmax to the last dimension (reference fused_ops.py:606-615)."""
    _require_cuda(x, "rational_softmax")
    return RationalSoftmax.apply(x, eps)


def rational_swiglu(gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """Apply the rational SwiGLU activation (reference fused_ops.py:618-626)."""
    _require_cuda(gate, "rational_swiglu")
    return RationalSwiGLU.apply(gate, value)


def add_mean_error_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = EPS):
    """(x + residual, mean_error_norm(x + residual, weight)) in one pass over the tensors."""
    _require_cuda(x, "add_mean_error_norm")
    return AddMeanErrorNorm.apply(x, residual, weight, eps)


def mean_error_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """Apply mean-error normalisation (reference fused_ops.py:629-636)."""
    _require_cuda(x, "mean_error_norm")
    return MeanErrorNorm.apply(x, weight, eps)
