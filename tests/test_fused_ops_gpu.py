"""Parity of the SwiGLU / mean-error-norm / rational-softmax kernels with the CPU oracle (B200)."""
import pytest
import torch

from conftest import bf16_violations, load_golden, norm_max_err
from oracle import oracle

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5      # max|a-b| / max|b|, the bar for float32
DEV = "cuda"


def fat():
    import fastalgebraictransformer_b200 as m
    return m


def run(fn, inputs, d_out):
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    out.backward(d_out.to(DEV))
    return out.detach(), [t.grad for t in leaves]


def gen(seed, *shapes, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(*s, generator=g) * std).to(dtype) for s in shapes]


def compare(got, want, dtype, what, f64_tol=1e-12):
    if dtype in (torch.float32, torch.float64):
        tol = FP32_TOL if dtype == torch.float32 else f64_tol
        assert norm_max_err(got, want) < tol, f"{what}: {norm_max_err(got, want):.3e}"
    else:   # bf16 / fp16: |a-b| <= 1e-2 + 2e-2 |b| on every element
        bad, nme = bf16_violations(got.float(), want)
        assert bad == 0.0, f"{what}: {bad:.2e} of elements outside rel 2e-2 / abs 1e-2 (norm max err {nme:.2e})"


def oracle_inputs(ts, dtype):
    """Low-precision inputs are rounded first, then the oracle runs in float32 on the rounded values."""
    up = torch.float64 if dtype == torch.float64 else torch.float32
    return [t.to(dtype).to(up) for t in ts]


# ----------------------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("tag", ["a", "b"])
def test_softmax_golden(tag):
    g = load_golden(f"softmax_{tag}")
    out, (dx,) = run(fat().rational_softmax, [g["x"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < FP32_TOL and norm_max_err(dx, g["dx"]) < FP32_TOL


@pytest.mark.parametrize("tag", ["a", "b"])
def test_swiglu_golden(tag):
    g = load_golden(f"swiglu_{tag}")
    out, (dg, dv) = run(fat().rational_swiglu, [g["gate"], g["value"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < FP32_TOL
    assert norm_max_err(dg, g["dgate"]) < FP32_TOL and norm_max_err(dv, g["dvalue"]) < FP32_TOL


@pytest.mark.parametrize("tag", ["a", "b"])
def test_norm_golden(tag):
    g = load_golden(f"norm_{tag}")
    out, (dx, dw) = run(fat().mean_error_norm, [g["x"], g["weight"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < FP32_TOL
    assert norm_max_err(dx, g["dx"]) < FP32_TOL and norm_max_err(dw, g["dweight"]) < FP32_TOL


# ----------------------------------------------------------------------------- seeded sweeps vs the oracle
SOFTMAX_SHAPES = [(2, 8, 64, 64), (4, 12, 128, 128), (2, 16, 256, 256),          # the reference's test shapes
                  (1, 1), (3, 1), (5, 7), (4, 37), (33, 1000), (3, 2048), (2, 4096), (2, 16384), (1, 20000), (2, 40000)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", SOFTMAX_SHAPES)
def test_softmax_vs_oracle(shape, dtype):
    x, go = gen(11, shape, shape, dtype=dtype)
    x = x * 2
    out, (dx,) = run(fat().rational_softmax, [x], go)
    xo, goo = oracle_inputs([x, go], dtype)
    want, (wdx,) = oracle.autograd_grads(oracle.rational_softmax, [xo], goo)
    compare(out, want, dtype, "softmax out")
    if shape[-1] == 1:
        # one column: p = f/(f+eps), the gradient is ~eps*d_out, the difference of two nearly equal numbers;
        # a relative bar is meaningless there, so it is checked absolutely
        assert (dx.double().cpu() - wdx.double()).abs().max() < 1e-5
    else:
        compare(dx, wdx, dtype, "softmax dx")
    if dtype == torch.float32 and shape[-1] >= 16:   # (rows of one tiny sigma^4 sum to f/(f+eps) < 1, as in the oracle)
        assert (out.sum(-1) - 1).abs().max().item() < 1e-5


SWIGLU_SHAPES = [(2, 512, 768), (4, 1024, 1024), (1, 1), (3, 5), (7, 33), (129, 2048), (2, 3, 1000)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", SWIGLU_SHAPES)
def test_swiglu_vs_oracle(shape, dtype):
    gate, val, go = gen(12, shape, shape, shape, dtype=dtype)
    out, (dg, dv) = run(fat().rational_swiglu, [gate, val], go)
    a, b, c = oracle_inputs([gate, val, go], dtype)
    want, (wdg, wdv) = oracle.autograd_grads(oracle.rational_swiglu, [a, b], c)
    compare(out, want, dtype, "swiglu out")
    compare(dg, wdg, dtype, "swiglu dgate")
    compare(dv, wdv, dtype, "swiglu dvalue")


def test_swiglu_reads_packed_halves_in_place():
    """gate / value as the two halves of one [rows, 2*ffn] projection (the model's layout)."""
    (gv, go) = gen(13, (4, 96, 2 * 344), (4, 96, 344))
    gv_d = gv.to(DEV).requires_grad_(True)
    gate, val = gv_d.chunk(2, dim=-1)
    out = fat().rational_swiglu(gate, val)
    out.backward(go.to(DEV))
    ref = gv.clone().requires_grad_(True)
    a, b = ref.chunk(2, dim=-1)
    oracle.rational_swiglu(a, b).backward(go)
    assert norm_max_err(out, oracle.rational_swiglu(a, b)) < FP32_TOL
    assert norm_max_err(gv_d.grad, ref.grad) < FP32_TOL


NORM_SHAPES = [(2, 512, 768), (4, 1024, 1024), (1, 1), (2, 3), (7, 50), (300, 2048), (64, 4096), (5, 8192), (3, 20000)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_norm_vs_oracle(shape, dtype):
    x, go = gen(14, shape, shape, dtype=dtype)
    (w,) = gen(15, (shape[-1],), dtype=dtype)
    w = (1 + 0.1 * w.float()).to(dtype)
    out, (dx, dw) = run(fat().mean_error_norm, [x, w], go)
    a, b, c = oracle_inputs([x, w, go], dtype)
    want, (wdx, wdw) = oracle.autograd_grads(oracle.mean_error_norm, [a, b], c)
    compare(out, want, dtype, "norm out")
    if shape[-1] == 1:
        # y = x/(|x|+eps)*w: the gradient w.r.t. x is ~eps, a cancellation; checked absolutely
        assert (dx.double().cpu() - wdx.double()).abs().max() < 1e-4
    else:
        # the backward reads the float32 row mean the forward saved (as the reference does), so a
        # float64 run cannot be closer than float32 rounding of that statistic
        compare(dx, wdx, dtype, "norm dx", f64_tol=1e-6)
    if dtype in (torch.float32, torch.float64):
        compare(dw, wdw, dtype, "norm dweight", f64_tol=1e-6)
    else:   # a column sum over many rows, rounded once to 16 bits at the end
        assert norm_max_err(dw.float(), wdw) < 1e-2


def run_add_norm(x, r, w, d_h, d_y):
    """(h, y, dx, dr, dw) of the fused residual addition + norm on the GPU."""
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (x, r, w)]
    h, y = fat().add_mean_error_norm(*leaves)
    torch.autograd.backward([h, y], [d_h.to(DEV), d_y.to(DEV)])
    return h.detach(), y.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad


@pytest.mark.parametrize("tag", ["a", "b"])
def test_add_norm_golden(tag):
    g = load_golden(f"add_norm_{tag}")
    got = run_add_norm(g["x"], g["residual"], g["weight"], g["d_h"], g["d_y"])
    for t, key in zip(got, ("h", "y", "dx", "dresidual", "dweight")):
        assert norm_max_err(t, g[key]) < FP32_TOL, key


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", [(2, 512, 768), (2, 3), (7, 50), (300, 2048), (64, 4096), (3, 20000)])
def test_add_norm_equals_the_two_separate_operators(shape, dtype):
    """The fused pass rounds the sum to the tensor dtype before normalising it and rounds the norm gradient before
    adding the residual gradient, exactly as the two separate passes do: bit-identical results, every dtype, including
    the shapes that fall back to the generic kernels."""
    x, r, d_h, d_y = gen(41, shape, shape, shape, shape, dtype=dtype)
    (w,) = gen(42, (shape[-1],), dtype=dtype)
    w = (1 + 0.1 * w.float()).to(dtype)
    h, y, dx, dr, dw = run_add_norm(x, r, w, d_h, d_y)
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (x, r, w)]
    h2 = leaves[0] + leaves[1]
    y2 = fat().mean_error_norm(h2, leaves[2])
    torch.autograd.backward([h2, y2], [d_h.to(DEV), d_y.to(DEV)])
    assert torch.equal(h, h2.detach()) and torch.equal(y, y2.detach())
    assert torch.equal(dx, leaves[0].grad) and torch.equal(dr, leaves[1].grad) and torch.equal(dw, leaves[2].grad)


def test_add_norm_only_one_result_used():
    """Gradients when only the sum or only the normalised sum feeds the loss."""
    x, r, d = gen(43, (6, 256), (6, 256), (6, 256))
    (w,) = gen(44, (256,))
    for use_h in (True, False):
        leaves = [t.to(DEV).requires_grad_(True) for t in (x, r, w)]
        h, y = fat().add_mean_error_norm(*leaves)
        ((h if use_h else y) * d.to(DEV)).sum().backward()
        ref = [t.clone().requires_grad_(True) for t in (x, r, w)]
        ho, yo = oracle.add_mean_error_norm(*ref)
        ((ho if use_h else yo) * d).sum().backward()
        assert norm_max_err(leaves[0].grad, ref[0].grad) < FP32_TOL and norm_max_err(leaves[1].grad, ref[1].grad) < FP32_TOL
        if use_h:
            assert leaves[2].grad is None or float(leaves[2].grad.abs().max()) == 0.0
        else:
            assert norm_max_err(leaves[2].grad, ref[2].grad) < FP32_TOL


# ----------------------------------------------------------------------------- shifted cross-entropy (loss head)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 32, 128), (3, 17, 1000), (2, 9, 1001), (1, 2, 8), (2, 5, 32000), (1, 3, 50000), (4, 1, 64)])
def test_shifted_cross_entropy_vs_oracle(shape, dtype):
    """Loss and d(loss)/d(logits) against the reference's own formulation (algebraic_model.py:229-235) in float32 on the
    rounded logits; some targets are ignore_index, T = 1 leaves nothing to score.  Covers the register-cached rows, the
    rows that are re-read (odd V, float32 rows wider than the cache) and a non-unit incoming gradient."""
    B, T, V = shape
    g = torch.Generator().manual_seed(51)
    logits = (torch.randn(B, T, V, generator=g) * 3).to(dtype)
    labels = torch.randint(0, V, (B, T), generator=g)
    labels[torch.rand(B, T, generator=g) < 0.2] = -100
    leaf = logits.to(DEV).requires_grad_(True)
    loss = fat().shifted_cross_entropy(leaf, labels.to(DEV), -100)
    (loss.float() * 3.0).backward()
    ref = logits.float().requires_grad_(True)
    want = oracle.shifted_cross_entropy(ref, labels, -100)
    if T == 1 or bool((labels[:, 1:] == -100).all()):
        assert float(loss.detach()) == 0.0 and float(leaf.grad.abs().max()) == 0.0      # the reference gives nan here (0/0)
        return
    (want * 3.0).backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert abs(float(loss.detach()) - float(want.detach())) <= tol * max(1.0, abs(float(want.detach())))
    gerr = (leaf.grad.float().cpu() - ref.grad).abs().max() / ref.grad.abs().max()
    assert gerr < (1e-5 if dtype == torch.float32 else 1e-2), gerr
    assert float(leaf.grad[:, -1].abs().max()) == 0.0                       # the last position is never scored


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 100, 32000), (2, 160, 50000), (8, 64, 1000), (3, 128, 8)])
def test_shifted_cross_entropy_many_rows_vs_oracle(shape, dtype):
    """Enough rows (at least two per SM) for the kernel that stages whole rows in shared memory: three, two and four rows
    in flight per CTA (64 KB, 100 KB and short rows), targets that are ignored, rows that only get zeros, a non-unit
    incoming gradient.  Loss and every element of the gradient against the float32 oracle on the rounded logits."""
    B, T, V = shape
    g = torch.Generator().manual_seed(53)
    logits = (torch.randn(B, T, V, generator=g) * 3).to(dtype)
    labels = torch.randint(0, V, (B, T), generator=g)
    labels[torch.rand(B, T, generator=g) < 0.2] = -100
    leaf = logits.to(DEV).requires_grad_(True)
    loss = fat().shifted_cross_entropy(leaf, labels.to(DEV), -100)
    (loss.float() * 3.0).backward()
    ref = logits.float().requires_grad_(True)
    want = oracle.shifted_cross_entropy(ref, labels, -100)
    (want * 3.0).backward()
    assert abs(float(loss.detach()) - float(want.detach())) <= 1e-2 * max(1.0, abs(float(want.detach())))
    got = leaf.grad.float().cpu()
    # per element: rel 2e-2 of the value plus an absolute floor far below the largest gradients (1/n_valid ~ 1e-3)
    assert ((got - ref.grad).abs() <= 2e-2 * ref.grad.abs() + 2e-2 * ref.grad.abs().max()).all()
    assert ((got - ref.grad).abs().max() / ref.grad.abs().max()).item() < 1e-2
    assert float(leaf.grad[:, -1].abs().max()) == 0.0                       # the last position is never scored
    ignored = labels[:, 1:] == -100
    assert float(leaf.grad[:, :-1][ignored.to(DEV)].abs().max()) == 0.0     # nor are ignored targets


def test_shifted_cross_entropy_in_place_and_strided_on_the_staged_kernel():
    """Through the C ABI, with enough rows for the staged kernel: the gradient written over the logits themselves gives
    the same bits as a separate gradient buffer, and so do logits read through a token stride."""
    from fastalgebraictransformer_b200 import _lib
    lib = _lib.lib()
    B, T, V = 4, 96, 32000
    g = torch.Generator().manual_seed(54)
    logits = (torch.randn(B, T, V, generator=g) * 2).to(torch.bfloat16).to(DEV)
    labels = torch.randint(0, V, (B, T), generator=g).to(DEV)
    n_valid = torch.tensor([float(B * (T - 1))], device=DEV)

    def run(src, ls_b, ls_t, dst):
        row_loss = torch.empty(B * T, device=DEV)
        rc = lib.fat_shifted_ce_fwd(src.data_ptr(), labels.data_ptr(), n_valid.data_ptr(), row_loss.data_ptr(), dst.data_ptr(), B, T, V,
                                    ls_b, ls_t, labels.stride(0), labels.stride(1), -100, _lib.BF16, _lib.stream_ptr(logits.device))
        assert rc == 0, lib.fat_last_error().decode()
        torch.cuda.synchronize()
        return row_loss

    grad = torch.empty_like(logits)
    loss_a = run(logits, T * V, V, grad)
    over = logits.clone()
    loss_b = run(over, T * V, V, over)                                      # gradient over the logits
    assert torch.equal(loss_a, loss_b) and torch.equal(grad, over)
    wide = torch.zeros(B, T, 2, V, dtype=torch.bfloat16, device=DEV)        # every second row of a wider buffer
    wide[:, :, 0] = logits
    grad_c = torch.empty_like(logits)
    loss_c = run(wide, T * 2 * V, 2 * V, grad_c)
    assert torch.equal(loss_a, loss_c) and torch.equal(grad, grad_c)


def test_shifted_cross_entropy_strided_logits_and_unit_gradient():
    """Logits that are a view with a token stride (as a head applied to a padded buffer would give) and the plain
    loss.backward() path, where the gradient is used exactly as the forward wrote it."""
    g = torch.Generator().manual_seed(52)
    big = torch.randn(2, 12, 256, generator=g)
    labels = torch.randint(0, 256, (2, 6), generator=g)
    view = big.to(DEV)[:, ::2, :].requires_grad_(True)
    assert not view.is_contiguous()
    loss = fat().shifted_cross_entropy(view, labels.to(DEV))
    (gr,) = torch.autograd.grad(loss, view)
    ref = big[:, ::2, :].clone().requires_grad_(True)
    want = oracle.shifted_cross_entropy(ref, labels)
    want.backward()
    assert abs(float(loss.detach()) - float(want.detach())) < 1e-5 * float(want.detach())
    assert norm_max_err(gr, ref.grad) < FP32_TOL


def test_norm_weight_randn_like_reference_test():
    """tests.py:141-173 draws the weight from randn; thresholds fwd 1e-4, grads 1e-3 (max abs)."""
    x, go = gen(16, (4, 1024, 1024), (4, 1024, 1024))
    (w,) = gen(17, (1024,))
    out, (dx, dw) = run(fat().mean_error_norm, [x, w], go)
    want, (wdx, wdw) = oracle.autograd_grads(oracle.mean_error_norm, [x, w], go)
    assert (out.cpu() - want).abs().max() < 1e-4
    assert (dx.cpu() - wdx).abs().max() < 1e-3 and ((dw.cpu() - wdw).abs().max() / wdw.abs().max()) < 1e-5


def test_norm_sign_of_zero_is_zero():
    x = torch.zeros(2, 64); x[:, ::2] = 1.5
    go = torch.ones(2, 64)
    w = torch.full((64,), 2.0)
    _, (dx, _) = run(fat().mean_error_norm, [x, w], go)
    _, (wdx, _) = oracle.autograd_grads(oracle.mean_error_norm, [x, w], go)
    assert norm_max_err(dx, wdx) < FP32_TOL


def test_empty_inputs():
    f = fat()
    e = torch.empty(0, 16, device=DEV)
    assert f.rational_softmax(e).shape == (0, 16)
    assert f.rational_swiglu(e, e).shape == (0, 16)
    assert f.mean_error_norm(e, torch.ones(16, device=DEV)).shape == (0, 16)


def test_gradcheck_float64():
    """The reference's gradcheck settings (tests.py:219-270): eps 1e-6, atol 1e-4, rtol 1e-3."""
    f = fat()
    g = torch.Generator().manual_seed(18)
    kw = dict(eps=1e-6, atol=1e-4, rtol=1e-3)
    x = torch.randn(2, 4, 16, 16, generator=g, dtype=torch.float64).to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(lambda t: f.RationalSoftmax.apply(t, 1e-6), (x,), **kw)
    gate = torch.randn(2, 16, 32, generator=g, dtype=torch.float64).to(DEV).requires_grad_(True)
    val = torch.randn(2, 16, 32, generator=g, dtype=torch.float64).to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(f.RationalSwiGLU.apply, (gate, val), **kw)
    x = torch.randn(2, 16, 32, generator=g, dtype=torch.float64).to(DEV).requires_grad_(True)
    w = torch.randn(32, generator=g, dtype=torch.float64).to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(lambda a, b: f.MeanErrorNorm.apply(a, b, 1e-6), (x, w), **kw)


def test_torch_library_ops_have_autograd():
    x = torch.randn(8, 64, device=DEV, requires_grad=True)
    y = torch.ops.algebraic.softmax_fwd(x, 1e-6)
    y.sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape


def test_full_size_properties():
    """Benchmark sizes, checked through size-independent properties instead of the (slow) oracle."""
    f = fat()
    g = torch.Generator(device=DEV).manual_seed(19)
    x = (torch.randn(4096, 4096, generator=g, device=DEV) * 1.4142).to(torch.bfloat16)
    p = f.rational_softmax(x)
    assert (p.float().sum(-1) - 1).abs().max().item() < 2e-2 and (p >= 0).all()
    xn = torch.randn(16384, 4096, generator=g, device=DEV).to(torch.bfloat16)
    w = torch.ones(4096, device=DEV, dtype=torch.bfloat16)
    y = f.mean_error_norm(xn, w)
    assert (y.float().abs().mean(-1) - 1).abs().max().item() < 1e-2            # rows have unit mean |y|
    y2 = f.mean_error_norm(2 * xn, w)                                            # scale invariance up to eps/mean
    assert (y2 != y).float().mean().item() < 1e-2 and (y2.float() - y.float()).abs().max().item() < 0.05
    gate = torch.randn(2048, 8192, generator=g, device=DEV).to(torch.bfloat16)
    val = torch.randn(2048, 8192, generator=g, device=DEV).to(torch.bfloat16)
    o1 = f.rational_swiglu(gate, val)
    assert torch.equal(f.rational_swiglu(gate, 2 * val), 2 * o1)                 # linear in value
    assert torch.equal(f.rational_swiglu(gate, val), o1)                         # deterministic


def _bar16(got, want, what):
    """Every element within |a-b| <= 1e-2 + 2e-2 |b| of the float32 oracle (the 16-bit bar)."""
    bad, nme = bf16_violations(got.float(), want)
    assert bad == 0.0, f"{what}: {bad:.2e} of elements outside the bar (norm max err {nme:.2e})"


def test_config3_swiglu_full_size_vs_oracle():
    """Bandwidth-sweep configuration, SwiGLU [16384, 8192] bf16 forward + backward, every element against the float32
    oracle on the rounded inputs (evaluated 2048 rows at a time to keep the host's working set small)."""
    g = torch.Generator().manual_seed(1234 + 2)
    gate, val, go = (torch.randn(16384, 8192, generator=g).to(torch.bfloat16) for _ in range(3))
    a, b = gate.to(DEV).requires_grad_(True), val.to(DEV).requires_grad_(True)
    out = fat().rational_swiglu(a, b)
    out.backward(go.to(DEV))
    got = [t.cpu() for t in (out.detach(), a.grad, b.grad)]
    for r0 in range(0, 16384, 2048):
        sl = slice(r0, r0 + 2048)
        want_out, (wg, wv) = oracle.autograd_grads(oracle.rational_swiglu, [gate[sl].float(), val[sl].float()], go[sl].float())
        for t, w, name in zip(got, (want_out, wg, wv), ("out", "d_gate", "d_value")):
            _bar16(t[sl], w, f"swiglu {name} rows {r0}..")


def test_config3_norm_full_size_vs_oracle():
    """Mean-error norm [16384, 4096] bf16 with weight 1 + 0.1 N(0,1): y, d_x and d_weight against the float32 oracle."""
    g = torch.Generator().manual_seed(1234 + 2)
    x = torch.randn(16384, 4096, generator=g).to(torch.bfloat16)
    go = torch.randn(16384, 4096, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(4096, generator=g)).to(torch.bfloat16)
    a, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    y = fat().mean_error_norm(a, wd)
    y.backward(go.to(DEV))
    want_y, (wx, ww) = oracle.autograd_grads(oracle.mean_error_norm, [x.float(), w.float()], go.float())
    _bar16(y.detach().cpu(), want_y, "norm y")
    _bar16(a.grad.cpu(), wx, "norm d_x")
    # d_weight sums 16384 rows: its magnitude is ~sqrt(16384), so the bar is applied relative to that scale
    assert norm_max_err(wd.grad, ww) < 2e-2


@pytest.mark.parametrize("std", [1.4142135, 2.0])
def test_config3_softmax_full_size_vs_oracle(std):
    """Rational softmax [4096, 4096] bf16, scores ~ N(0, 2) read both ways (variance 2 and standard deviation 2)."""
    g = torch.Generator().manual_seed(1234 + 2)
    x = (torch.randn(4096, 4096, generator=g) * std).to(torch.bfloat16)
    go = torch.randn(4096, 4096, generator=g).to(torch.bfloat16)
    a = x.to(DEV).requires_grad_(True)
    p = fat().rational_softmax(a)
    p.backward(go.to(DEV))
    want_p, (wx,) = oracle.autograd_grads(oracle.rational_softmax, [x.float()], go.float())
    _bar16(p.detach().cpu(), want_p, "softmax p")
    _bar16(a.grad.cpu(), wx, "softmax d_x")
    assert norm_max_err(p.detach().float().cpu(), want_p) < 2e-2 and norm_max_err(a.grad.float().cpu(), wx) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 32, 64, 128), (3, 17, 32, 1000), (2, 64, 128, 32000)])
def test_head_loss_without_logits_vs_oracle(shape, dtype):
    """The loss head for callers that do not keep the logits: loss, d_y and d_weight of cross_entropy((y W^T)[:, :-1],
    labels[:, 1:]) with the logits existing one sequence at a time, against the reference's formulation in float32, and
    against this library's own two-step path (head GEMM, then the loss over the full logits)."""
    B, T, C, V = shape
    g = torch.Generator().manual_seed(53)
    y = torch.randn(B, T, C, generator=g).to(dtype)
    w = (torch.randn(V, C, generator=g) * 0.3).to(dtype)
    labels = torch.randint(0, V, (B, T), generator=g)
    labels[torch.rand(B, T, generator=g) < 0.2] = -100
    yd, wd = y.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    loss = fat().head_shifted_cross_entropy(yd, wd, labels.to(DEV), -100)
    (loss.float() * 2.0).backward()
    yr, wr = y.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    want = oracle.shifted_cross_entropy(yr @ wr.t(), labels, -100)
    (want * 2.0).backward()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert abs(float(loss.detach()) - float(want.detach())) <= tol * max(1.0, abs(float(want.detach())))
    assert norm_max_err(yd.grad, yr.grad) < (2e-5 if dtype == torch.float32 else 2e-2)
    assert norm_max_err(wd.grad, wr.grad) < (2e-5 if dtype == torch.float32 else 2e-2)
    # the two-step path of the same library
    y2, w2 = y.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    loss2 = fat().shifted_cross_entropy(y2 @ w2.t(), labels.to(DEV), -100)
    (loss2.float() * 2.0).backward()
    assert abs(float(loss.detach()) - float(loss2.detach())) <= tol * max(1.0, abs(float(want.detach())))
    assert norm_max_err(yd.grad, y2.grad.cpu()) < (2e-5 if dtype == torch.float32 else 2e-2)
    with torch.no_grad():                              # loss only: no gradient buffers, same number
        loss3 = fat().head_shifted_cross_entropy(y.to(DEV), w.to(DEV), labels.to(DEV), -100)
    assert float(loss3) == float(loss.detach())
