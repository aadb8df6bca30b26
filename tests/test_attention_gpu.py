"""Parity of the rational-attention kernels with the CPU oracle and the golden vectors (B200)."""
import math

import pytest
import torch

from conftest import bf16_violations, load_golden, norm_max_err
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP32_TOL = 1e-5


def fat():
    import fastalgebraictransformer_b200 as m
    return m


def run_attention(q, k, v, go, slopes, scale, causal=True, path=0, eps=1e-6):
    from fastalgebraictransformer_b200.backward import RationalAttentionFunction
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = RationalAttentionFunction.apply(*leaves, slopes.to(DEV), scale, causal, eps, path, False)
    out.backward(go.to(DEV))
    fat().check_device_status()
    return out.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad


def gen_qkv(seed, B, H, T, D, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, T, D, generator=g).to(dtype) for _ in range(4)]


@pytest.mark.parametrize("tag", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("path", [1])
def test_golden_fp32(tag, path):
    g = load_golden(f"attention_{tag}")
    out, dq, dk, dv = run_attention(g["q"], g["k"], g["v"], g["d_out"], g["slopes"], g["scale"], path=path)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert norm_max_err(got, g[key]) < FP32_TOL, f"{key}: {norm_max_err(got, g[key]):.2e}"
        # the reference's own thresholds (tests.py:210-211): fwd < 1e-3, grads < 1e-2 max abs
        assert (got.cpu() - g[key]).abs().max() < (1e-3 if key == "out" else 1e-2)


SHAPES = [(1, 1, 1, 8), (1, 2, 2, 16), (2, 3, 17, 32), (1, 2, 63, 64), (1, 2, 64, 64), (1, 2, 65, 64), (1, 4, 127, 32),
          (1, 2, 129, 128), (2, 2, 200, 40), (1, 1, 300, 100), (1, 12, 256, 64)]


@pytest.mark.parametrize("shape", SHAPES)
def test_fp32_vs_oracle(shape):
    B, H, T, D = shape
    q, k, v, go = gen_qkv(21, B, H, T, D)
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    out, dq, dk, dv = run_attention(q, k, v, go, slopes, scale, path=1)
    want = oracle.rational_attention_grads(q, k, v, go, slopes, scale)
    for got, w, name in zip((out, dq, dk, dv), want, ("out", "dq", "dk", "dv")):
        if T == 1 and name in ("dq", "dk"):
            # a single key: dS = k (dP - Delta) / (L+eps) is ~eps, the difference of two equal numbers
            assert (got.cpu() - w).abs().max() < 1e-5
        else:
            assert norm_max_err(got, w) < FP32_TOL, f"{name}: {norm_max_err(got, w):.2e}"


def test_config1_fp32_closed_form_slopes():
    """Benchmark configuration 1: B=2,H=12,S=512,D=64 float32, slopes 2^(-8(i+1)/12)."""
    B, H, T, D = 2, 12, 512, 64
    g = torch.Generator().manual_seed(1234 + 0)
    q, k, v, go = (torch.randn(B, H, T, D, generator=g) for _ in range(4))
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)])
    out, dq, dk, dv = run_attention(q, k, v, go, slopes, 0.125)
    want = oracle.rational_attention_grads(q, k, v, go, slopes, 0.125)
    for got, w, name in zip((out, dq, dk, dv), want, ("out", "dq", "dk", "dv")):
        assert norm_max_err(got, w) < FP32_TOL, f"{name}: {norm_max_err(got, w):.2e}"
    # and once with the library's own slopes for 12 heads (not a power of two)
    slopes = fat().compute_alibi_slopes(12)
    out = run_attention(q, k, v, go, slopes, 0.125)[0]
    assert norm_max_err(out, oracle.rational_attention(q, k, v, slopes, 0.125)) < FP32_TOL


def test_forward_returns_row_sums_without_eps():
    B, H, T, D = 1, 2, 70, 32
    q, k, v, _ = gen_qkv(22, B, H, T, D)
    slopes = oracle.compute_alibi_slopes(H)
    out, L = fat().rational_attention_forward(q.to(DEV), k.to(DEV), v.to(DEV), slopes.to(DEV), 0.2)
    assert L.dtype == torch.float32 and L.shape == (B, H, T)
    assert norm_max_err(L, oracle.rational_attention_rowsum(q, k, slopes, 0.2)) < FP32_TOL
    assert norm_max_err(out, oracle.rational_attention(q, k, v, slopes, 0.2)) < FP32_TOL


def test_explicit_backward_entry_point():
    B, H, T, D = 1, 2, 50, 32
    q, k, v, go = gen_qkv(23, B, H, T, D)
    slopes = oracle.compute_alibi_slopes(H)
    f = fat()
    qd, kd, vd, god, sd = (t.to(DEV) for t in (q, k, v, go, slopes))
    out, L = f.rational_attention_forward(qd, kd, vd, sd, 0.3)
    dq, dk, dv = f.rational_attention_backward(qd, kd, vd, out, L, god, sd, 0.3)
    want = oracle.rational_attention_grads(q, k, v, go, slopes, 0.3)
    for got, w in zip((dq, dk, dv), want[1:]):
        assert norm_max_err(got, w) < FP32_TOL


def test_non_causal_extension():
    """causal=False has no reference behaviour; checked against the oracle with its mask line removed."""
    B, H, T, D = 1, 2, 90, 32
    q, k, v, go = gen_qkv(24, B, H, T, D)
    slopes = oracle.compute_alibi_slopes(H)
    out, dq, dk, dv = run_attention(q, k, v, go, slopes, 0.2, causal=False, path=1)
    want = oracle.rational_attention_grads(q, k, v, go, slopes, 0.2, causal=False)
    for got, w in zip((out, dq, dk, dv), want):
        assert norm_max_err(got, w) < FP32_TOL


def test_strided_views_of_packed_projection():
    """q, k, v as the model passes them: permuted views of one [B,T,3,H,D] buffer (algebraic_model.py:89-91)."""
    B, H, T, D = 2, 4, 96, 32
    g = torch.Generator().manual_seed(25)
    packed = torch.randn(B, T, 3, H, D, generator=g)
    go = torch.randn(B, H, T, D, generator=g)
    slopes = oracle.compute_alibi_slopes(H)
    pd = packed.to(DEV).requires_grad_(True)
    q, k, v = pd.permute(2, 0, 3, 1, 4).unbind(0)
    assert not q.is_contiguous()
    out = fat().rational_attention(q, k, v, slopes.to(DEV), 0.2)
    out.backward(go.to(DEV))
    pr = packed.clone().requires_grad_(True)
    qr, kr, vr = pr.permute(2, 0, 3, 1, 4).unbind(0)
    ref = oracle.rational_attention(qr, kr, vr, slopes, 0.2)
    ref.backward(go)
    assert norm_max_err(out, ref) < FP32_TOL and norm_max_err(pd.grad, pr.grad) < FP32_TOL


def assert_16bit_bar(got, want, what=""):
    """Every element of out, dq, dk, dv within |a-b| <= 1e-2 + 2e-2 |b| of the float32 oracle."""
    for g, w, name in zip(got, want, ("out", "dq", "dk", "dv")):
        bad, nme = bf16_violations(g.float(), w)
        assert not torch.isnan(g.float()).any(), f"{what}{name}: NaN"
        assert bad == 0.0, f"{what}{name}: {bad:.2e} of elements outside the bar (norm max err {nme:.2e})"


# the last two are the attention shapes of the small LM (12 heads: slopes that are no powers of one base, D=64, T=1024)
# and of the XL LM (16 heads, D=128, T=2048)
# (1, 4, 192, 64), (2, 2, 320, 128), (1, 2, 176, 64): a last tile of 33..64 rows, where two of the backward's four
# 32-row d_q quarters lie beyond T
LOWP_SHAPES = [(1, 2, 64, 64), (2, 4, 200, 64), (1, 2, 333, 128), (1, 3, 100, 32), (1, 16, 512, 128),
               (8, 12, 1024, 64), (1, 16, 2048, 128), (1, 4, 192, 64), (2, 2, 320, 128), (1, 2, 176, 64)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", LOWP_SHAPES)
@pytest.mark.parametrize("path", [0, 1, 3])
def test_low_precision_vs_oracle(shape, dtype, path):
    """bf16 / fp16: inputs rounded, oracle in float32 on the rounded values, bar rel 2e-2 / abs 1e-2 on every element
    of the output and of the three gradients, for the fused tensor-core kernels (0), the CUDA-core kernels (1) and the
    deterministic tensor-core pair (3)."""
    B, H, T, D = shape
    if path == 3 and D not in (64, 128):
        pytest.skip("no tensor-core kernel for this head size")
    if path == 1 and B * H * T >= 8 * 12 * 1024 and dtype == torch.float16:
        pytest.skip("the CUDA-core kernels are covered on this shape in bf16")
    q, k, v, go = gen_qkv(26, B, H, T, D, dtype)
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    got = run_attention(q, k, v, go, slopes, scale, path=path)
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go.float(), slopes, scale)
    assert_16bit_bar(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("path", [0, 3])
@pytest.mark.parametrize("gscale", [1e-6, 1e-2, 1e2, 1e4, 1e6])
def test_gradient_magnitude_does_not_matter(dtype, path, gscale):
    """d_out as a loss scaler or a late-training step leaves it: the tensor-core backward stores dS as float16 scaled by
    a power of two taken from max|d_out| of the (batch, head), so the gradients are d_out-homogeneous - finite, and
    inside the bar after dividing the scale out again."""
    B, H, T, D = 1, 4, 300, 128
    q, k, v, go = gen_qkv(41, B, H, T, D, dtype)
    if dtype == torch.float16 and not 1e-3 < gscale < 1e3:
        pytest.skip("d_out or the gradients themselves would leave float16's range")
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    go_scaled = (go.float() * gscale).to(dtype)
    out, dq, dk, dv = run_attention(q, k, v, go_scaled, slopes, scale, path=path)
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go_scaled.float() / gscale, slopes, scale)
    for g in (dq, dk, dv):
        assert torch.isfinite(g.float()).all()
    assert_16bit_bar((out, dq.float() / gscale, dk.float() / gscale, dv.float() / gscale), want, f"x{gscale:g} ")


def test_bf16_inputs_beyond_float16_are_reported():
    """The tensor-core backward works on float16 copies of q and k.  A bfloat16 magnitude of 65536 or more does not fit:
    the kernel clamps it and says so in the status word; the CUDA-core path takes such tensors."""
    B, H, T, D = 1, 2, 256, 64
    q, k, v, go = gen_qkv(42, B, H, T, D, torch.bfloat16)
    k[0, 1, 200, 3] = 1.0e5
    slopes = oracle.compute_alibi_slopes(H)
    with pytest.raises(RuntimeError, match="65536"):
        run_attention(q, k, v, go, slopes, 0.125, path=2)
    got = run_attention(q, k, v, go, slopes, 0.125, path=1)
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go.float(), slopes, 0.125)
    assert_16bit_bar(got, want)


@pytest.mark.parametrize("shape", [(2, 4, 333, 64), (1, 16, 700, 128), (2, 12, 1024, 64)])
def test_packed_projection_bf16_tensor_path(shape):
    """The model's layout on the tensor cores: q, k, v read in place from one [B,T,3,H,D] projection through strided
    tensor maps, the output written token-major, the three gradients landing in one packed buffer
    (algebraic_model.py:89-107) - against the oracle on the permuted views."""
    from fastalgebraictransformer_b200.backward import RationalAttentionPackedFunction
    B, H, T, D = shape
    g = torch.Generator().manual_seed(43)
    packed = torch.randn(B, T, 3, H, D, generator=g).to(torch.bfloat16)
    go = torch.randn(B, T, H * D, generator=g).to(torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    pd = packed.to(DEV).requires_grad_(True)
    out = RationalAttentionPackedFunction.apply(pd, slopes.to(DEV), scale, 1e-6)
    assert out.shape == (B, T, H * D) and out.is_contiguous()
    out.backward(go.to(DEV))
    fat().check_device_status()
    q, k, v = packed.float().permute(2, 0, 3, 1, 4).unbind(0)
    want = oracle.rational_attention_grads(q, k, v, go.float().view(B, T, H, D).permute(0, 2, 1, 3), slopes, scale)
    got_out = out.detach().view(B, T, H, D).permute(0, 2, 1, 3)
    gq, gk, gv = pd.grad.permute(2, 0, 3, 1, 4).unbind(0)
    assert_16bit_bar((got_out, gq, gk, gv), want)


def test_deterministic():
    """The CUDA-core path and the deterministic tensor path (no atomics anywhere): two runs give bit-identical outputs
    and gradients."""
    from fastalgebraictransformer_b200 import PATH_SIMT, PATH_TENSOR_DETERMINISTIC
    B, H, T, D = 1, 4, 300, 64
    q, k, v, go = gen_qkv(27, B, H, T, D, torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    for path in (PATH_SIMT, PATH_TENSOR_DETERMINISTIC):
        a = run_attention(q, k, v, go, slopes, 0.125, path=path)
        b = run_attention(q, k, v, go, slopes, 0.125, path=path)
        assert all(torch.equal(x, y) for x, y in zip(a, b)), path


@pytest.mark.parametrize("D", [64, 128])
def test_deterministic_tensor_path(D):
    """The default tensor-core backward accumulates d_q across key tiles with reduce-adds (order varies between runs, so
    its last bits may); path 3 selects the two-kernel backward, which is bit-reproducible."""
    from fastalgebraictransformer_b200 import PATH_TENSOR_DETERMINISTIC
    B, H, T = 1, 4, 700
    q, k, v, go = gen_qkv(29, B, H, T, D, torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    a = run_attention(q, k, v, go, slopes, 0.09, path=PATH_TENSOR_DETERMINISTIC)
    b = run_attention(q, k, v, go, slopes, 0.09, path=PATH_TENSOR_DETERMINISTIC)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    c = run_attention(q, k, v, go, slopes, 0.09)              # fused backward
    for x, y, name in zip(a, c, ("out", "dq", "dk", "dv")):
        if name == "out":
            assert torch.equal(x, y)
        else:
            assert norm_max_err(x.float(), y.float().cpu()) < 1e-2, name
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go.float(), slopes, 0.09)
    assert_16bit_bar(c, want, "fused ")
    assert_16bit_bar(a, want, "deterministic ")


@pytest.mark.parametrize("T", [640, 1280, 1408])
@pytest.mark.parametrize("D", [64, 128])
def test_tile_counts_that_leave_padding_blocks(T, D):
    """The causal kernels run on 1-D grids ordered in bands of tile ranks; tile counts that are no multiple of the band
    size (here odd numbers of query blocks in the forward's two bands) leave padding blocks that must return without
    touching anything, and every real tile must still be visited exactly once.  Tensor path against the CUDA-core path."""
    B, H = 1, 3
    q, k, v, go = gen_qkv(31 + T // 128, B, H, T, D, torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    tc = run_attention(q, k, v, go, slopes, scale, path=2)
    simt = run_attention(q, k, v, go, slopes, scale, path=1)
    for a, b, name in zip(tc, simt, ("out", "dq", "dk", "dv")):
        assert not torch.isnan(a.float()).any(), name
        assert norm_max_err(a.float(), b.float().cpu()) < 1.5e-2, name


def test_tensor_core_path_agrees_with_cuda_core_path():
    """The two kernel families against each other on the device (bf16, D=128, ragged T)."""
    B, H, T, D = 2, 4, 777, 128
    q, k, v, go = gen_qkv(28, B, H, T, D, torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    tc = run_attention(q, k, v, go, slopes, 0.09, path=2)
    simt = run_attention(q, k, v, go, slopes, 0.09, path=1)
    for a, b, name in zip(tc, simt, ("out", "dq", "dk", "dv")):
        assert norm_max_err(a.float(), b.float().cpu()) < 1.5e-2, name


def test_forced_tensor_path_rejects_ineligible_requests():
    q = torch.randn(1, 2, 64, 32, device=DEV, dtype=torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(2).to(DEV)
    with pytest.raises(RuntimeError):
        torch.ops.algebraic.attn_fwd(q, q, q, slopes, 0.2, True, 1e-6, 2, False)      # D=32 has no tcgen05 kernel
    q = torch.randn(1, 2, 64, 64, device=DEV, dtype=torch.float32)
    with pytest.raises(RuntimeError):
        torch.ops.algebraic.attn_fwd(q, q, q, slopes, 0.2, True, 1e-6, 2, False)      # float32 runs on the CUDA cores


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 64, 64), (2, 3, 200, 64), (1, 2, 333, 128), (1, 4, 512, 128), (1, 2, 192, 64), (1, 2, 1024, 128)])
@pytest.mark.parametrize("path", [2, 3])
def test_non_causal_on_the_tensor_cores(shape, dtype, path):
    """causal=False on the tcgen05 kernels (every query sees every key, bias -slope |i-j| on both sides of the diagonal,
    zero-filled keys of a ragged last tile masked): against the oracle with its mask line removed.  Parity unpinned by the
    reference for this flag: its kernels never read it."""
    B, H, T, D = shape
    q, k, v, go = gen_qkv(61, B, H, T, D, dtype)
    slopes = oracle.compute_alibi_slopes(H)
    scale = 1.0 / math.sqrt(D)
    got = run_attention(q, k, v, go, slopes, scale, causal=False, path=path)
    want = oracle.rational_attention_grads(q.float(), k.float(), v.float(), go.float(), slopes, scale, causal=False)
    assert_16bit_bar(got, want)


def test_config2_slice_bf16():
    """Benchmark configuration 2 (B=8,H=16,S=4096,D=128 bf16), one batch element against the oracle, the rest through
    a property: heads and batch elements are independent, so batch element b of the full run equals a run on it alone."""
    H, T, D = 16, 4096, 128
    g = torch.Generator().manual_seed(1234 + 1)
    q, k, v, go = (torch.randn(2, H, T, D, generator=g).to(torch.bfloat16) for _ in range(4))
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)])
    scale = 1.0 / math.sqrt(D)
    full = run_attention(q, k, v, go, slopes, scale)
    one = run_attention(q[1:], k[1:], v[1:], go[1:], slopes, scale)
    for a, b, name in zip(full, one, ("out", "dq", "dk", "dv")):
        if name == "dq":     # D=128: float32 reduce-adds across key tiles in an unordered sequence (last-bit differences)
            assert (a[1:] != b).float().mean().item() < 1e-2 and norm_max_err(a[1:].float(), b.float().cpu()) < 1e-2
        else:
            assert torch.equal(a[1:], b), name
    # all 16 heads of batch element 0 against the oracle, one head at a time (keeps the oracle's S x S temporaries small);
    # heads 8-15 have slopes <= 2^-4.5: row sums in the hundreds to thousands, every key contributes
    for h in range(H):
        sl = slice(h, h + 1)
        want = oracle.rational_attention_grads(q[:1, sl].float(), k[:1, sl].float(), v[:1, sl].float(), go[:1, sl].float(),
                                               slopes[sl], scale)
        assert_16bit_bar(tuple(t[:1, sl] for t in full), want, f"head {h} ")
    # the CUDA-core kernels meet the bar on the two steepest heads of the same batch element
    want = oracle.rational_attention_grads(q[:1, :2].float(), k[:1, :2].float(), v[:1, :2].float(), go[:1, :2].float(),
                                           slopes[:2], scale)
    got = run_attention(q[:1, :2], k[:1, :2], v[:1, :2], go[:1, :2], slopes[:2], scale, path=1)
    assert_16bit_bar(got, want, "simt ")
