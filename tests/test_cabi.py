"""The C-ABI library: it builds, loads, and exports exactly what include/fat_b200.h declares (no GPU)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def libpath():
    from fastalgebraictransformer_b200 import build
    return build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fat_b200.h")).read()
    return sorted(set(re.findall(r"FAT_API[^;(]*?\b(fat_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for want in ("fat_swiglu_fwd", "fat_swiglu_bwd", "fat_norm_fwd", "fat_norm_bwd", "fat_softmax_fwd",
                 "fat_softmax_bwd", "fat_attn_fwd", "fat_attn_bwd", "fat_attn_bwd_workspace_bytes",
                 "fat_norm_bwd_workspace_bytes"):
        assert want in names


def test_library_exports_every_declared_symbol(libpath):
    handle = ctypes.CDLL(libpath)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in fat_b200.h but not exported"


def test_binding_covers_every_declared_symbol(libpath):
    from fastalgebraictransformer_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_symbols()
    lib = _lib.lib()
    assert lib.fat_version() >= 100
    assert lib.fat_error_string(0) == b"ok"


def test_host_side_argument_errors_need_no_gpu(libpath):
    """Shape / dtype / null validation happens before any CUDA call."""
    from fastalgebraictransformer_b200 import _lib
    lib = _lib.lib()
    assert lib.fat_swiglu_fwd(None, None, None, 4, 0, 0, 0, 0, _lib.F32, None) == 2          # bad shape
    assert lib.fat_swiglu_fwd(None, None, None, 4, 8, 8, 8, 8, _lib.F32, None) == 7          # null pointer
    assert lib.fat_swiglu_fwd(None, None, None, 0, 8, 8, 8, 8, _lib.F32, None) == 0          # empty: nothing to do
    assert lib.fat_softmax_fwd(ctypes.c_void_p(16), ctypes.c_void_p(16), 1, 8, 8, 8, 1e-6, 99, None) == 1   # dtype
    assert b"dtype" in lib.fat_last_error()
    s3 = (ctypes.c_int64 * 3)(1, 1, 1)
    assert lib.fat_attn_fwd(None, None, None, None, None, None, None, 1, 0, 4, 8, s3, s3, s3, s3, 1.0, 1e-6, 1,
                            _lib.F32, 0, None, None) == 2
    assert lib.fat_attn_fwd(None, None, None, None, None, None, None, 1, 2, 4, 8, s3, s3, s3, s3, 1.0, 1e-6, 1,
                            _lib.F64, 0, None, None) == 1
    assert lib.fat_norm_bwd_workspace_bytes(10, 4096, _lib.BF16) == 2 * 148 * 4096 * 4   # 2 blocks per SM, 148 SMs (a B200; also assumed when no device answers)
    assert lib.fat_attn_bwd_workspace_bytes(2, 3, 5, 64, _lib.F32, _lib.PATH_SIMT) == 2 * 3 * 5 * 4
    # padding-mask and decode entry points: sizes and argument errors are decided on the host
    assert [lib.fat_key_mask_words(t) for t in (0, 1, 128, 129, 4096)] == [0, 4, 4, 8, 128]
    assert lib.fat_pack_key_mask(None, None, 2, 16, 16, 1, None) == 7
    assert lib.fat_pack_key_mask(None, None, 0, 16, 16, 1, None) == 0
    assert lib.fat_attn_fwd_masked(None, None, None, None, None, None, None, None, 1, 0, 4, 8, s3, s3, s3, s3, 1.0, 1e-6, 1,
                                   _lib.F32, 0, None, None) == 2
    s2 = (ctypes.c_int64 * 2)(1, 1)
    assert lib.fat_attn_decode(None, None, None, None, None, None, None, None, 1, 2, 0, 64, s2, s2, s2, s2, s3, s3, 1.0, 1e-6,
                               _lib.F32, None, None) == 2
    assert lib.fat_attn_decode(None, None, None, None, None, None, None, None, 1, 2, 16, 64, s2, s2, s2, s2, s3, s3, 1.0, 1e-6,
                               _lib.F32, None, None) == 7


def test_cpu_tensors_are_rejected_not_emulated(libpath):
    import torch
    import fastalgebraictransformer_b200 as fat
    x = torch.randn(4, 8)
    with pytest.raises(RuntimeError):
        fat.rational_softmax(x)
    with pytest.raises(RuntimeError):
        fat.rational_swiglu(x, x)
    with pytest.raises(RuntimeError):
        fat.mean_error_norm(x, torch.ones(8))
    q = torch.randn(1, 2, 4, 8)
    with pytest.raises(RuntimeError):
        fat.rational_attention(q, q, q, fat.compute_alibi_slopes(2), 1.0)


def test_reference_import_names():
    """The reference's tests import the package as ``kernels`` with these sub-modules."""
    import kernels
    from kernels.fused_ops import rational_softmax, rational_swiglu, mean_error_norm, RationalSoftmax, RationalSwiGLU, MeanErrorNorm  # noqa
    from kernels.forward import rational_attention_forward, compute_alibi_slopes  # noqa
    from kernels.backward import rational_attention, rational_attention_backward, RationalAttentionFunction  # noqa
    from kernels.algebraic_model import AlgebraicTransformerLM, create_small_model  # noqa
    assert kernels.EPS == 1e-6 and kernels.RationalSwiGLUModule is kernels.algebraic_model.RationalSwiGLU


def test_alibi_slopes_match_golden():
    import torch
    from conftest import load_golden
    import fastalgebraictransformer_b200 as fat
    g = load_golden("alibi_slopes")
    for h in (1, 2, 4, 6, 8, 12, 16, 24, 40):
        assert torch.allclose(fat.compute_alibi_slopes(h), g[f"h{h}"], rtol=1e-6, atol=0)


def test_build_module_imports_without_the_libraries():
    """`python -m fastalgebraictransformer_b200.build` has to work in a fresh checkout: importing the package and its build
    module must not touch the operator library (the public names load it on first use)."""
    import subprocess
    import sys
    code = ("import sys; import fastalgebraictransformer_b200 as f; from fastalgebraictransformer_b200 import build; "
            "assert 'fastalgebraictransformer_b200.ops' not in sys.modules; "
            "assert 'rational_attention' in dir(f) and callable(build.build); print('ok')")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-500:]
