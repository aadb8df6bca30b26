"""The give-up path of the bounded waits, run once in the allowed form.

Every wait inside the tcgen05 kernels is bounded: when the bound is hit the kernel records a status word, raises a CTA-wide
flag that makes all later waits fall through, and runs to its normal teardown (named barriers, TMEM release).  Nothing in
normal operation makes a wait run out, so a TEST-ONLY build of the library (tests/_build/libfat_b200_waittest.so, made by
`python -m fastalgebraictransformer_b200.build`; the package never loads it) compiles the attention forward with a
producer that leaves out one V tile and with waits that give up after ~3 ms.  One single-CTA launch of it must return by
itself with the status word set; an ordinary launch of the shipped library right after must be correct, which also shows
that the tensor memory of the SM was released.  No trap, no faulting access, no unbounded loop is involved.
"""
import ctypes
import math
import os

import pytest
import torch

from conftest import ROOT, bf16_violations
from oracle import oracle

pytestmark = pytest.mark.gpu
LIB = os.path.join(ROOT, "tests", "_build", "libfat_b200_waittest.so")


def test_a_wait_that_runs_out_ends_in_a_status_word_and_a_usable_gpu():
    if not os.path.exists(LIB):
        pytest.skip("tests/_build/libfat_b200_waittest.so has not been built")
    import fastalgebraictransformer_b200 as fat
    from fastalgebraictransformer_b200 import _lib
    dev = torch.device("cuda", 0)
    B, H, T, D = 1, 1, 128, 64
    g = torch.Generator().manual_seed(71)
    q, k, v, go = (torch.randn(B, H, T, D, generator=g).to(torch.bfloat16) for _ in range(4))
    slopes = oracle.compute_alibi_slopes(H)
    qd, kd, vd, sd = (t.to(dev) for t in (q, k, v, slopes))
    out = torch.empty_like(qd)
    out_lo = torch.empty_like(qd)
    L = torch.empty(B, H, T, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    test_lib = ctypes.CDLL(LIB)                                # its own handle: the symbols stay local to it
    fn = test_lib.fat_attn_fwd
    fn.restype, fn.argtypes = _lib.PROTOTYPES["fat_attn_fwd"]
    rc = fn(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), sd.data_ptr(), out.data_ptr(), out_lo.data_ptr(), L.data_ptr(),
            B, H, T, D, _lib.strides3(qd), _lib.strides3(kd), _lib.strides3(vd), _lib.strides3(out), 1.0 / math.sqrt(D), 1e-6,
            1, _lib.BF16, _lib.PATH_TENSOR, status.data_ptr(), _lib.stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()                                   # returns: the kernel ended by itself
    word = int(status.item())
    assert (word >> 24) & 0x1f == 1, f"status word 0x{word:08x}: expected the wait-timeout code"
    assert word & 0xffffff in (22, 23, 30, 31, 40, 10, 11), f"status word 0x{word:08x}: unexpected wait site"

    # the shipped library on the same GPU, right after: correct results (and no kernel stuck waiting for tensor memory)
    leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    res = fat.rational_attention(*leaves, sd, 1.0 / math.sqrt(D))
    res.backward(go.to(dev))
    fat.check_device_status()
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go.float(), slopes, 1.0 / math.sqrt(D))
    for got, w in zip((res, leaves[0].grad, leaves[1].grad, leaves[2].grad), want):
        bad, _ = bf16_violations(got.float(), w)
        assert bad == 0.0
