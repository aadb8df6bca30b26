"""The CPU oracle against the golden vectors generated from the reference (no GPU needed).

These tests pin ``oracle/oracle.py``: every restated function must reproduce what the
reference's own PyTorch functions produced for the saved, seeded inputs.
"""
import pytest
import torch

from conftest import load_golden, norm_max_err
from oracle import oracle

TOL = 2e-6     # same arithmetic, same library: only re-association noise is allowed


@pytest.mark.parametrize("h", [1, 2, 4, 6, 8, 12, 16, 24, 40])
def test_alibi_slopes(h):
    g = load_golden("alibi_slopes")
    assert torch.allclose(oracle.compute_alibi_slopes(h), g[f"h{h}"], rtol=1e-6, atol=0)


def test_alibi_closed_form_for_power_of_two():
    for h in (2, 4, 8, 16, 32):
        want = torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)])
        assert torch.allclose(oracle.compute_alibi_slopes(h), want, rtol=1e-6)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_softmax(tag):
    g = load_golden(f"softmax_{tag}")
    out, (dx,) = oracle.autograd_grads(oracle.rational_softmax, [g["x"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < TOL
    assert norm_max_err(dx, g["dx"]) < TOL
    assert norm_max_err(oracle.rational_softmax_grad(g["x"], g["d_out"]), g["dx"]) < 2e-5
    assert (out.sum(-1) - 1).abs().max() < 1e-5


@pytest.mark.parametrize("tag", ["a", "b"])
def test_swiglu(tag):
    g = load_golden(f"swiglu_{tag}")
    out, (dg, dv) = oracle.autograd_grads(oracle.rational_swiglu, [g["gate"], g["value"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < TOL
    assert norm_max_err(dg, g["dgate"]) < TOL and norm_max_err(dv, g["dvalue"]) < TOL
    cg, cv = oracle.rational_swiglu_grad(g["gate"], g["value"], g["d_out"])
    assert norm_max_err(cg, g["dgate"]) < 1e-5 and norm_max_err(cv, g["dvalue"]) < 1e-5


@pytest.mark.parametrize("tag", ["a", "b"])
def test_norm(tag):
    g = load_golden(f"norm_{tag}")
    out, (dx, dw) = oracle.autograd_grads(oracle.mean_error_norm, [g["x"], g["weight"]], g["d_out"])
    assert norm_max_err(out, g["out"]) < TOL
    assert norm_max_err(dx, g["dx"]) < TOL and norm_max_err(dw, g["dweight"]) < TOL
    cx, cw = oracle.mean_error_norm_grad(g["x"], g["weight"], g["d_out"])
    assert norm_max_err(cx, g["dx"]) < 1e-5 and norm_max_err(cw, g["dweight"]) < 1e-5
    assert norm_max_err(g["x"].abs().mean(-1), g["mean"]) < TOL


@pytest.mark.parametrize("tag", ["a", "b"])
def test_add_norm(tag):
    """Residual addition + norm as the reference's block composes them; both results carry a gradient."""
    g = load_golden(f"add_norm_{tag}")
    leaves = [g[k].clone().requires_grad_(True) for k in ("x", "residual", "weight")]
    h, y = oracle.add_mean_error_norm(*leaves)
    ((h * g["d_h"]).sum() + (y * g["d_y"]).sum()).backward()
    assert norm_max_err(h.detach(), g["h"]) < TOL and norm_max_err(y.detach(), g["y"]) < TOL
    for leaf, key in zip(leaves, ("dx", "dresidual", "dweight")):
        assert norm_max_err(leaf.grad, g[key]) < TOL, key


@pytest.mark.parametrize("tag", ["a", "b", "c", "d", "e"])
def test_attention(tag):
    g = load_golden(f"attention_{tag}")
    args = (g["q"], g["k"], g["v"], g["d_out"], g["slopes"], g["scale"])
    out, dq, dk, dv = oracle.rational_attention_grads(*args)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert norm_max_err(got, g[key]) < TOL, key
    # the closed form the kernels implement (eps-free gradient factor)
    out, dq, dk, dv = oracle.rational_attention_grads_closed_form(*args)
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert norm_max_err(got, g[key]) < 1e-5, key
    L = oracle.rational_attention_rowsum(g["q"], g["k"], g["slopes"], g["scale"])
    assert L.shape == g["q"].shape[:3] and (L > 0).all()
    # the last query row on its own (what a key/value-cached decode step computes) is the reference's last row
    last = oracle.rational_attention_last_row(g["q"][:, :, -1], g["k"], g["v"], g["slopes"], g["scale"])
    assert norm_max_err(last, g["out"][:, :, -1]) < TOL


@pytest.mark.parametrize("tag", ["a", "b"])
def test_attention_with_padding_mask(tag):
    """The oracle's key mask against the reference's masked attention (its model's PyTorch path)."""
    g = load_golden(f"attention_masked_{tag}")
    out, dq, dk, dv = oracle.rational_attention_grads(g["q"], g["k"], g["v"], g["d_out"], g["slopes"], g["scale"],
                                                       key_mask=g["mask"])
    for got, key in ((out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert norm_max_err(got, g[key]) < TOL, key


def test_lm_tiny_with_padding_mask():
    g, m = load_golden("lm_tiny"), load_golden("lm_tiny_masked")
    state = {k[3:].replace("__", "."): v for k, v in g.items() if k.startswith("w__")}
    state["head.weight"] = state.pop("embed.weight")
    logits, loss = oracle.lm_forward(state, g["input_ids"], g["n_head"], g["labels"], attention_mask=m["attention_mask"])
    assert norm_max_err(logits, m["logits"]) < 1e-5
    assert abs(loss.item() - m["loss"]) < 1e-5


def test_lm_tiny():
    g = load_golden("lm_tiny")
    state = {k[3:].replace("__", "."): v for k, v in g.items() if k.startswith("w__")}
    state["head.weight"] = state.pop("embed.weight")
    logits, loss = oracle.lm_forward(state, g["input_ids"], g["n_head"], g["labels"])
    assert norm_max_err(logits, g["logits"]) < 1e-5
    assert abs(loss.item() - g["loss"]) < 1e-5
    loss2, grads = oracle.lm_loss_and_grads(state, g["input_ids"], g["labels"], g["n_head"])
    grads["embed.weight"] = grads.pop("head.weight")
    for k, v in g.items():
        if k.startswith("g__"):
            assert norm_max_err(grads[k[3:].replace("__", ".")], v) < 2e-5, k
