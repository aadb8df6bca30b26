"""Generate the golden vectors in this directory from the reference implementation.

Run once, in a checkout that has the reference's sources next to it:

    python tests/golden/make_golden.py --reference /path/to/parent/of/reference

The reference package is imported as ``reference`` (its own ``tests.py`` holds the
PyTorch reference functions, tests.py:20-65; the language model runs on the CPU through
its built-in fallbacks, algebraic_model.py:37-39, 57-60, 102-136).  Inputs are seeded,
evaluated in float32 on the CPU, and saved together with the outputs and the autograd
gradients, so that the fixtures can be checked anywhere without the reference.
"""
import argparse
import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


ONLY = None       # set by --only: write just the fixtures whose name starts with this prefix


def save(name, **arrays):
    if ONLY and not name.startswith(ONLY):
        return
    out = {k: (v.detach().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in arrays.items()}
    np.savez(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: tuple(v.shape) for k, v in out.items()})


def grads(fn, inputs, d_out):
    leaves = [t.clone().requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    out.backward(d_out)
    return out.detach(), [t.grad for t in leaves]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that contains the 'reference' package")
    ap.add_argument("--only", default=None, help="write only the fixtures whose name starts with this prefix")
    args = ap.parse_args()
    global ONLY
    ONLY = args.only
    sys.path.insert(0, args.reference)
    ref_tests = importlib.import_module("reference.tests")
    ref_fwd = importlib.import_module("reference.forward")
    ref_model = importlib.import_module("reference.algebraic_model")
    torch.set_num_threads(1)

    # --- ALiBi slopes for every head count the tests and configs use (forward.py:21-42)
    save("alibi_slopes", **{f"h{h}": ref_fwd.compute_alibi_slopes(h) for h in (1, 2, 4, 6, 8, 12, 16, 24, 40)})

    # --- rational softmax: reference test shape (2,8,64,64) trimmed to (2,2,64,64), plus a ragged row
    g = torch.Generator().manual_seed(101)
    for tag, shape, std in (("a", (2, 2, 64, 64), 1.0), ("b", (3, 37), 2.0)):
        x = torch.randn(*shape, generator=g) * std
        go = torch.randn(*shape, generator=g)
        out, (dx,) = grads(ref_tests.ref_rational_softmax, [x], go)
        save(f"softmax_{tag}", x=x, d_out=go, out=out, dx=dx)

    # --- rational SwiGLU
    g = torch.Generator().manual_seed(102)
    for tag, shape in (("a", (2, 16, 96)), ("b", (5, 33))):
        gate = torch.randn(*shape, generator=g)
        val = torch.randn(*shape, generator=g)
        go = torch.randn(*shape, generator=g)
        out, (dg, dv) = grads(ref_tests.ref_rational_swiglu, [gate, val], go)
        save(f"swiglu_{tag}", gate=gate, value=val, d_out=go, out=out, dgate=dg, dvalue=dv)

    # --- mean-error norm (weight ~ randn as in tests.py:146)
    g = torch.Generator().manual_seed(103)
    for tag, shape in (("a", (2, 16, 96)), ("b", (7, 50))):
        x = torch.randn(*shape, generator=g)
        w = torch.randn(shape[-1], generator=g)
        go = torch.randn(*shape, generator=g)
        out, (dx, dw) = grads(ref_tests.ref_mean_error_norm, [x, w], go)
        save(f"norm_{tag}", x=x, weight=w, d_out=go, out=out, dx=dx, dweight=dw,
             mean=x.abs().mean(-1))

    # --- residual addition followed by the norm, as a pre-norm block does it (algebraic_model.py:149-152): both the sum
    #     and the normalised sum are used downstream, so both receive a gradient
    g = torch.Generator().manual_seed(107)
    for tag, shape in (("a", (2, 16, 96)), ("b", (7, 50))):
        x = torch.randn(*shape, generator=g)
        r = torch.randn(*shape, generator=g)
        w = torch.randn(shape[-1], generator=g)
        d_h = torch.randn(*shape, generator=g)
        d_y = torch.randn(*shape, generator=g)
        leaves = [t.clone().requires_grad_(True) for t in (x, r, w)]
        h = leaves[0] + leaves[1]
        y = ref_tests.ref_mean_error_norm(h, leaves[2])
        ((h * d_h).sum() + (y * d_y).sum()).backward()
        save(f"add_norm_{tag}", x=x, residual=r, weight=w, d_h=d_h, d_y=d_y, h=h.detach(), y=y.detach(),
             dx=leaves[0].grad, dresidual=leaves[1].grad, dweight=leaves[2].grad)

    # --- attention: the reference's own test shapes (tests.py:183) and a ragged one
    g = torch.Generator().manual_seed(104)
    for tag, (B, H, T, D) in (("a", (1, 4, 32, 32)), ("b", (1, 8, 64, 64)), ("c", (1, 4, 128, 32)),
                              ("d", (1, 3, 77, 64)), ("e", (1, 1, 160, 128))):
        q, k, v, go = (torch.randn(B, H, T, D, generator=g) for _ in range(4))
        slopes = ref_fwd.compute_alibi_slopes(H)
        scale = 1.0 / D ** 0.5
        out, (dq, dk, dv) = grads(lambda a, b, c: ref_tests.ref_rational_attention(a, b, c, slopes, scale),
                                  [q, k, v], go)
        save(f"attention_{tag}", q=q, k=k, v=v, d_out=go, slopes=slopes, scale=np.float32(scale),
             out=out, dq=dq, dk=dk, dv=dv)

    # --- attention with a padding mask: the only place the reference applies one is the PyTorch path of its attention
    #     module (algebraic_model.py:112-136), so that method is what is recorded (scale 1/sqrt(D), the module's slopes)
    g = torch.Generator().manual_seed(107)
    for tag, (B, H, T, D), pads in (("a", (2, 4, 48, 32), ((40, 48), (0, 5))),              # right padding, left padding
                                    ("b", (3, 1, 136, 64), ((100, 136), (0, 0), (60, 131)))):  # ... none, and a hole
        q, k, v, go = (torch.randn(B, H, T, D, generator=g) for _ in range(4))
        mask = torch.ones(B, T, dtype=torch.int64)
        for b, (lo, hi) in enumerate(pads):
            mask[b, lo:hi] = 0
        attn = ref_model.AlgebraicAttention(d_model=H * D, n_head=H, dropout=0.0)
        out, (dq, dk, dv) = grads(lambda a, b, c: attn._cpu_attention(a, b, c, mask), [q, k, v], go)
        save(f"attention_masked_{tag}", q=q, k=k, v=v, d_out=go, mask=mask, slopes=attn.alibi_slopes, scale=np.float32(attn.scale),
             out=out, dq=dq, dk=dk, dv=dv)

    # --- language model: a shrunken version of the reference smoke test (tests.py:281-290), dropout 0
    torch.manual_seed(105)
    cfg = dict(vocab_size=128, d_model=64, n_head=4, n_layers=2)
    model = ref_model.AlgebraicTransformerLM(dropout=0.0, **cfg)
    model.train()
    g = torch.Generator().manual_seed(106)
    ids = torch.randint(0, cfg["vocab_size"], (2, 32), generator=g)
    labels = torch.randint(0, cfg["vocab_size"], (2, 32), generator=g)
    logits, loss = model(ids, labels=labels)
    loss.backward()
    named = [(n, p) for n, p in model.named_parameters()]
    save("lm_tiny", input_ids=ids, labels=labels, loss=loss.detach(), logits=logits.detach(),
         n_head=np.int64(cfg["n_head"]),
         **{"w__" + n.replace(".", "__"): p.detach() for n, p in named},
         **{"g__" + n.replace(".", "__"): p.grad for n, p in named})

    # --- the same model and inputs with a padding mask (weights as in lm_tiny; right padding and left padding)
    model.zero_grad()
    mask = torch.ones(2, 32, dtype=torch.int64)
    mask[0, 25:] = 0
    mask[1, :3] = 0
    logits, loss = model(ids, labels=labels, attention_mask=mask)
    loss.backward()
    save("lm_tiny_masked", attention_mask=mask, loss=loss.detach(), logits=logits.detach(),
         **{"g__" + n.replace(".", "__"): p.grad for n, p in named})


if __name__ == "__main__":
    main()
