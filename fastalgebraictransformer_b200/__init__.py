"""B200-native Algebraic Transformer hot path.

Same public names as the reference package (``__init__.py:7-63``); the implementation is
hand-written sm_100a CUDA behind a C ABI (``libfat_b200.so``, ``include/fat_b200.h``) and a C++
registration of the ``torch.ops.algebraic`` operators (``libfat_torch_ops.so``).

The names below are resolved on first use: touching any of them loads the two libraries and fails
loudly if they have not been built (there is no fallback implementation).  Importing the bare package,
or its ``build`` module (``python -m fastalgebraictransformer_b200.build``), needs neither library.
"""
import importlib as _importlib

_EXPORTS = {
    "rational_softmax": "fused_ops", "rational_swiglu": "fused_ops", "mean_error_norm": "fused_ops",
    "add_mean_error_norm": "fused_ops", "RationalSoftmax": "fused_ops", "RationalSwiGLU": "fused_ops",
    "MeanErrorNorm": "fused_ops", "AddMeanErrorNorm": "fused_ops", "ShiftedCrossEntropy": "fused_ops",
    "shifted_cross_entropy": "fused_ops", "HeadShiftedCrossEntropy": "fused_ops", "head_shifted_cross_entropy": "fused_ops",
    "EPS": "fused_ops",
    "rational_attention_forward": "forward", "compute_alibi_slopes": "forward",
    "rational_attention": "backward", "rational_attention_backward": "backward", "RationalAttentionFunction": "backward",
    "AlgebraicTransformerLM": "algebraic_model", "RationalMR": "algebraic_model", "AlgebraicAttention": "algebraic_model",
    "AlgebraicBlock": "algebraic_model", "create_small_model": "algebraic_model", "create_medium_model": "algebraic_model",
    "create_large_model": "algebraic_model", "create_xl_model": "algebraic_model",
    "check_device_status": "_lib", "PATH_AUTO": "_lib", "PATH_SIMT": "_lib", "PATH_TENSOR": "_lib",
    "PATH_TENSOR_DETERMINISTIC": "_lib",
}
# the reference exports the autograd Function as RationalSwiGLU and the module under this alias (__init__.py:31)
_ALIASES = {"RationalSwiGLUModule": ("algebraic_model", "RationalSwiGLU")}
_SUBMODULES = ("fused_ops", "forward", "backward", "algebraic_model", "ops", "_lib", "build")

__all__ = [
    "rational_softmax", "rational_swiglu", "mean_error_norm", "add_mean_error_norm", "RationalSoftmax", "RationalSwiGLU",
    "MeanErrorNorm", "AddMeanErrorNorm", "ShiftedCrossEntropy", "shifted_cross_entropy", "HeadShiftedCrossEntropy",
    "head_shifted_cross_entropy", "EPS",
    "rational_attention_forward", "compute_alibi_slopes",
    "rational_attention", "rational_attention_backward", "RationalAttentionFunction",
    "AlgebraicTransformerLM", "RationalMR", "AlgebraicAttention", "AlgebraicBlock",
    "create_small_model", "create_medium_model", "create_large_model", "create_xl_model",
]


def __getattr__(name):
    if name in _EXPORTS:
        value = getattr(_importlib.import_module("." + _EXPORTS[name], __name__), name)
    elif name in _ALIASES:
        mod, attr = _ALIASES[name]
        value = getattr(_importlib.import_module("." + mod, __name__), attr)
    elif name in _SUBMODULES:
        value = _importlib.import_module("." + name, __name__)
    else:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(_EXPORTS) | set(_ALIASES) | set(_SUBMODULES))
