"""Drop-in import name of the reference package (its tests and README import ``kernels``).

``kernels``, ``kernels.fused_ops``, ``kernels.forward``, ``kernels.backward`` and
``kernels.algebraic_model`` are the modules of ``fastalgebraictransformer_b200``.
"""
import sys as _sys

import fastalgebraictransformer_b200 as _impl
from fastalgebraictransformer_b200 import *  # noqa: F401,F403
from fastalgebraictransformer_b200 import RationalSwiGLUModule, __all__  # noqa: F401
from fastalgebraictransformer_b200 import algebraic_model, backward, forward, fused_ops  # noqa: F401

for _name in ("fused_ops", "forward", "backward", "algebraic_model"):
    _sys.modules[__name__ + "." + _name] = getattr(_impl, _name)
