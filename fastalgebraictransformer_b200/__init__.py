"""B200-native Algebraic Transformer hot path.

Same public names as the reference package (``__init__.py:7-63``); the implementation is
hand-written sm_100a CUDA behind a C ABI (``libfat_b200.so``, ``include/fat_b200.h``).
"""
from .fused_ops import (rational_softmax, rational_swiglu, mean_error_norm, add_mean_error_norm, RationalSoftmax,
                        RationalSwiGLU, MeanErrorNorm, AddMeanErrorNorm, ShiftedCrossEntropy, shifted_cross_entropy,
                        HeadShiftedCrossEntropy, head_shifted_cross_entropy, EPS)
from .forward import rational_attention_forward, compute_alibi_slopes
from .backward import rational_attention, rational_attention_backward, RationalAttentionFunction
from .algebraic_model import (AlgebraicTransformerLM, RationalMR, RationalSwiGLU as RationalSwiGLUModule,
                              AlgebraicAttention, AlgebraicBlock, create_small_model, create_medium_model,
                              create_large_model, create_xl_model)
from ._lib import check_device_status, PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_TENSOR_DETERMINISTIC

__all__ = [
    "rational_softmax", "rational_swiglu", "mean_error_norm", "add_mean_error_norm", "RationalSoftmax", "RationalSwiGLU",
    "MeanErrorNorm", "AddMeanErrorNorm", "ShiftedCrossEntropy", "shifted_cross_entropy", "HeadShiftedCrossEntropy",
    "head_shifted_cross_entropy", "EPS",
    "rational_attention_forward", "compute_alibi_slopes",
    "rational_attention", "rational_attention_backward", "RationalAttentionFunction",
    "AlgebraicTransformerLM", "RationalMR", "AlgebraicAttention", "AlgebraicBlock",
    "create_small_model", "create_medium_model", "create_large_model", "create_xl_model",
]
