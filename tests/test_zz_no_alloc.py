"""fat_norm_bwd_static: the mean-error-norm backward whose scratch lives inside the library.

Some callers of the C ABI cannot allocate device memory at call time (a plugin running inside
another framework's memory plan, a callback where cudaMalloc is off limits).  For them the
library offers a variant of the norm backward that keeps the d_weight partial sums in a fixed
16 MiB device array instead of a caller-owned workspace.  This file checks, through the C ABI,
that it returns what the ordinary entry point returns, twice in a row (the array keeps the
previous call's contents, so the second call proves nothing stale leaks through), and that it
refuses sizes beyond its capacity.  It is collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, _lib, static, go, x, w, mean, eps):
    n_rows, n_cols = x.shape
    d_x = torch.empty_like(x)
    d_w = torch.empty_like(w)
    stream = _lib.stream_ptr(x.device)
    tag = _lib.dtype_tag(x)
    if static:
        # the property the entry point exists for: between here and its return nothing is taken from the device,
        # neither through torch's caching allocator nor from the driver
        torch.cuda.synchronize()
        held, (free, _) = torch.cuda.memory_allocated(x.device), torch.cuda.mem_get_info(x.device)
        rc = lib.fat_norm_bwd_static(go.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), d_x.data_ptr(),
                                     d_w.data_ptr(), n_rows, n_cols, go.stride(0), x.stride(0), d_x.stride(0), eps, tag,
                                     stream)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(x.device) == held and torch.cuda.mem_get_info(x.device)[0] >= free
    else:
        nbytes = lib.fat_norm_bwd_workspace_bytes(n_rows, n_cols, tag)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        rc = lib.fat_norm_bwd(go.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), d_x.data_ptr(), d_w.data_ptr(),
                              ws.data_ptr(), nbytes, n_rows, n_cols, go.stride(0), x.stride(0), d_x.stride(0), eps, tag,
                              stream)
    assert rc == 0, lib.fat_last_error().decode()
    torch.cuda.synchronize()
    return d_x, d_w


# the last two sit at the capacity of the built-in array on a 148-SM GPU (16 MiB / (296 blocks x 4 or 8 bytes))
@pytest.mark.parametrize("dtype,shape", [(torch.bfloat16, (4096, 4096)), (torch.float32, (300, 1000)),
                                         (torch.float32, (7, 50)), (torch.float32, (600, 14168)),
                                         (torch.float64, (600, 7084))])
def test_static_scratch_variant_matches_workspace_variant(dtype, shape):
    from fastalgebraictransformer_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    eps = 1e-6
    if lib.fat_norm_bwd_workspace_bytes(shape[0], shape[1], _lib.DTYPE_TAG[dtype]) > lib.fat_norm_bwd_static_capacity():
        pytest.skip("this GPU has more SMs than the case was sized for")
    for seed in (41, 42):                       # two calls in a row, different data
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(*shape, generator=g).to(dtype).to(dev)
        go = torch.randn(*shape, generator=g).to(dtype).to(dev)
        w = (1 + 0.1 * torch.randn(shape[1], generator=g)).to(dtype).to(dev)
        mean = x.float().abs().mean(-1).contiguous()
        want_dx, want_dw = _call(lib, _lib, False, go, x, w, mean, eps)
        got_dx, got_dw = _call(lib, _lib, True, go, x, w, mean, eps)
        # same kernels, same launch shape, same summation order: the results are bit-identical,
        # which is well inside the 16-bit (rel 2e-2 / abs 1e-2) and float32 (1e-5) bars used elsewhere
        assert torch.equal(got_dx, want_dx)
        assert torch.equal(got_dw, want_dw)


def test_static_scratch_variant_rejects_oversized_rows():
    from fastalgebraictransformer_b200 import _lib
    lib = _lib.lib()
    assert lib.fat_norm_bwd_static_capacity() == 16 << 20
    p = ctypes.c_void_p(256)
    rc = lib.fat_norm_bwd_static(p, p, p, p, p, p, 8, 32768, 32768, 32768, 32768, 1e-6, _lib.F32, None)
    assert rc == 5 and b"built-in array" in lib.fat_last_error()
