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


def test_a_copy_that_never_arrives_ends_in_nan_losses_and_a_usable_gpu():
    """The staged loss kernel: in the test build the first block never requests the copy of its fifth row.  The wait for
    it runs out (~3 ms), the block marks its rows with NaN losses, every block returns, and the shipped library gives the
    right loss on the same GPU right after."""
    if not os.path.exists(LIB):
        pytest.skip("tests/_build/libfat_b200_waittest.so has not been built")
    import fastalgebraictransformer_b200 as fat
    from fastalgebraictransformer_b200 import _lib
    dev = torch.device("cuda", 0)
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    B, T, V = 4, 2 * n_sm, 4096                                # 8 rows per block: enough for the staged kernel, and for row 4 of block 0
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(B, T, V, generator=g).to(torch.bfloat16)
    labels = torch.randint(0, V, (B, T), generator=g)
    ld, lab = logits.to(dev), labels.to(dev)
    n_valid = torch.tensor([float(B * (T - 1))], device=dev)
    row_loss = torch.zeros(B * T, device=dev)
    d_logits = torch.empty_like(ld)

    test_lib = ctypes.CDLL(LIB)
    fn = test_lib.fat_shifted_ce_fwd
    fn.restype, fn.argtypes = _lib.PROTOTYPES["fat_shifted_ce_fwd"]
    rc = fn(ld.data_ptr(), lab.data_ptr(), n_valid.data_ptr(), row_loss.data_ptr(), d_logits.data_ptr(), B, T, V, ld.stride(0), ld.stride(1),
            lab.stride(0), lab.stride(1), -100, _lib.BF16, _lib.stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()                                   # returns: every block ended by itself
    bad = torch.isnan(row_loss)
    mine = torch.arange(B * T, device=dev) % n_sm == 0         # the rows of block 0
    assert bad[mine].all() and not bad[~mine].any()

    want = oracle.shifted_cross_entropy(logits.float(), labels)
    got = fat.shifted_cross_entropy(ld, lab)
    assert abs(got.item() - want.item()) < 4e-2               # (the loss comes back in the logits' dtype: bfloat16 near 8.8 has steps of 0.06)
