"""CPU oracle for the Algebraic-Transformer hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic of the reference's
PyTorch reference path.  It exists so that the CUDA kernels can be checked against it;
it is never imported by the product package.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  Every function below is checked (tests/test_oracle_golden.py)
against golden vectors produced by importing the reference's own functions
(tests.py:20-65, forward.py:21-42, algebraic_model.py:155-237) with the generator
script tests/golden/make_golden.py.

Conventions
-----------
* Everything is evaluated in float32 (or float64 when the inputs are float64).  The
  reference's attention oracle cannot run in bf16 (it mixes an fp32 ALiBi bias with bf16
  values and torch.matmul refuses the mixed dtypes), so "the bf16 oracle" is this code
  evaluated on bf16-rounded inputs that were upcast to fp32.
* Gradients are offered twice: through autograd of the forward restatement (the
  reference's own definition of the gradient) and as closed forms.  The test-suite
  checks that both agree, which pins the formulae the kernels implement.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

EPS = 1e-6          # fused_ops.py:20
MASK_FILL = -1e4    # tests.py:59 (score given to masked positions)


# --------------------------------------------------------------------------------------
# element-wise pieces
# --------------------------------------------------------------------------------------

def rational_sigmoid(x: torch.Tensor) -> torch.Tensor:
    """sigma(x) = (x / (|x| + 1) + 1) / 2            (tests.py:20-22)."""
    return (x / (x.abs() + 1.0) + 1.0) * 0.5


def rational_softmax(x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """p = sigma(x)^4 / (sum_lastdim sigma(x)^4 + eps)   (tests.py:25-29)."""
    f = rational_sigmoid(x).pow(4)
    return f / (f.sum(dim=-1, keepdim=True) + eps)


def rational_swiglu(gate: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """out = gate * sigma(gate) * value                   (tests.py:32-35)."""
    return gate * rational_sigmoid(gate) * value


def mean_error_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """y = x / (mean_lastdim |x| + eps) * weight           (tests.py:38-41)."""
    m = x.abs().mean(dim=-1, keepdim=True)
    return x / (m + eps) * weight


def add_mean_error_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = EPS):
    """(h, y): h = x + residual, y = mean_error_norm(h, weight) — the residual addition of a pre-norm block
    and the normalisation that follows it (algebraic_model.py:149-152, with the norm of 26-39)."""
    h = x + residual
    return h, mean_error_norm(h, weight, eps)


def shifted_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """The language-model loss exactly as the reference writes it (algebraic_model.py:229-235)."""
    shift_logits = logits[..., :-1, :].contiguous()
    shift_labels = labels[..., 1:].contiguous()
    return torch.nn.functional.cross_entropy(shift_logits.view(-1, shift_logits.size(-1)), shift_labels.view(-1),
                                             ignore_index=ignore_index)


def compute_alibi_slopes(n_heads: int) -> torch.Tensor:
    """ALiBi slopes (forward.py:21-42).

    For a power-of-two head count n the slopes are 2^(-8 (i+1)/n).  Otherwise the slopes
    of the largest power of two p <= n are followed by the odd-indexed slopes of 2p.
    """
    def geometric(n: int, idx) -> torch.Tensor:
        base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return torch.pow(base, torch.as_tensor(list(idx)))

    p = 2 ** int(math.floor(math.log2(n_heads)))
    out = geometric(p, range(1, p + 1))
    if p != n_heads:
        extra = min(p, n_heads - p)
        out = torch.cat([out, geometric(2 * p, range(1, 1 + 2 * extra, 2))])
    return out.float()


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------

def _scores(q, k, slopes, scale, causal=True, key_mask=None):
    """scores = q k^T * scale - slope_h |i-j|, masked entries set to -1e4 (tests.py:48-59).  ``key_mask`` [B, T]: keys
    whose entry is 0 are padding and are filled the same way, as the reference's model does on its PyTorch path
    (algebraic_model.py:128-131)."""
    B, H, T, D = q.shape
    s = torch.matmul(q, k.transpose(-2, -1)) * scale
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).abs().to(torch.float32)
    s = s + (-dist * slopes.view(1, H, 1, 1).to(torch.float32)).to(s.dtype)
    if causal:
        future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
        s = s.masked_fill(future[None, None], MASK_FILL)
    if key_mask is not None:
        s = s.masked_fill(key_mask[:, None, None, :] == 0, MASK_FILL)
    return s


def rational_attention(q, k, v, slopes, scale, eps: float = EPS, causal: bool = True, key_mask=None):
    """Causal rational attention with ALiBi (tests.py:44-65).

    ``causal=False`` is this oracle's natural extension (mask line removed); the
    reference never defines it (its kernels and its own oracle are always causal).
    """
    return torch.matmul(rational_softmax(_scores(q, k, slopes, scale, causal, key_mask), eps), v)


def rational_attention_last_row(q, k, v, slopes, scale, eps: float = EPS):
    """Row T-1 of ``rational_attention`` computed on its own: q [B,H,D] is the query of the newest token, k, v [B,H,T,D]
    hold every token including it.  The same arithmetic as tests.py:44-65 restricted to the last query row (nothing is
    masked for it), i.e. what one step of a key/value-cached generate() needs; the reference itself recomputes all rows
    (algebraic_model.py:239-265)."""
    B, H, T, D = k.shape
    s = torch.einsum("bhd,bhtd->bht", q, k) * scale
    dist = (T - 1 - torch.arange(T)).to(torch.float32)
    s = s + (-dist[None, None] * slopes.view(1, H, 1).to(torch.float32)).to(s.dtype)
    return torch.einsum("bht,bhtd->bhd", rational_softmax(s, eps), v)


def rational_attention_rowsum(q, k, slopes, scale, causal: bool = True):
    """L_i = sum_j sigma(s_ij)^4 without eps — the statistic the forward launcher returns
    next to the output (forward.py:150-159)."""
    return rational_sigmoid(_scores(q, k, slopes, scale, causal)).pow(4).sum(-1)


def rational_attention_grads(q, k, v, d_out, slopes, scale, eps: float = EPS, causal: bool = True, key_mask=None):
    """(out, dq, dk, dv) via autograd through the forward restatement, one batch element at
    a time so that S=4096 fits in host memory."""
    outs, dqs, dks, dvs = [], [], [], []
    for b in range(q.shape[0]):
        qb, kb, vb = (t[b:b + 1].detach().clone().requires_grad_(True) for t in (q, k, v))
        o = rational_attention(qb, kb, vb, slopes, scale, eps, causal, None if key_mask is None else key_mask[b:b + 1])
        o.backward(d_out[b:b + 1])
        outs.append(o.detach()); dqs.append(qb.grad); dks.append(kb.grad); dvs.append(vb.grad)
    return tuple(torch.cat(t, 0) for t in (outs, dqs, dks, dvs))


def rational_attention_grads_closed_form(q, k, v, d_out, slopes, scale, eps: float = EPS,
                                         causal: bool = True):
    """Closed-form gradients: the algebra of backward.py:7-46 with the eps-free factor.

        r = 1/(|s|+1), sigma = (s r + 1)/2, f = sigma^4, p = f/(L+eps)
        dP_ij = dO_i . v_j,  Delta_i = dO_i . O_i
        dS_ij = 2 sigma^3 r^2 (dP_ij - Delta_i) / (L_i + eps)
        dQ = scale dS K,  dK = scale dS^T Q,  dV = P^T dO
    """
    s = _scores(q, k, slopes, scale, causal)
    r = 1.0 / (s.abs() + 1.0)
    sig = (s * r + 1.0) * 0.5
    f = sig.pow(4)
    inv = 1.0 / (f.sum(-1, keepdim=True) + eps)
    p = f * inv
    out = p @ v
    dp = d_out @ v.transpose(-2, -1)
    delta = (d_out * out).sum(-1, keepdim=True)
    ds = 2.0 * sig.pow(3) * r * r * (dp - delta) * inv
    if causal:
        T = q.shape[2]
        future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
        ds = ds.masked_fill(future[None, None], 0.0)
    return out, scale * (ds @ k), scale * (ds.transpose(-2, -1) @ q), p.transpose(-2, -1) @ d_out


# --------------------------------------------------------------------------------------
# closed-form gradients of the fused ops
# --------------------------------------------------------------------------------------

def rational_softmax_grad(x, d_out, eps: float = EPS):
    """dx = 2 sigma^3 r^2 / (Z+eps) * (dOut - sum(dOut p)), the algebra of
    fused_ops.py:113-150 with the eps-free factor."""
    r = 1.0 / (x.abs() + 1.0)
    sig = (x * r + 1.0) * 0.5
    f = sig.pow(4)
    inv = 1.0 / (f.sum(-1, keepdim=True) + eps)
    dot = (d_out * f * inv).sum(-1, keepdim=True)
    return 2.0 * sig.pow(3) * r * r * inv * (d_out - dot)


def rational_swiglu_grad(gate, value, d_out):
    """(dgate, dvalue) = (dOut value (sigma + gate sigma'), dOut gate sigma),
    sigma' = 1/(2 (|gate|+1)^2)                    (fused_ops.py:236-288)."""
    r = 1.0 / (gate.abs() + 1.0)
    sig = (gate * r + 1.0) * 0.5
    return d_out * value * (sig + gate * 0.5 * r * r), d_out * gate * sig


def mean_error_norm_grad(x, weight, d_out, eps: float = EPS):
    """(dx, dweight) with mu = mean|x| + eps  (fused_ops.py:349-423, 593-597):
        dx = dOut w / mu - sign(x) (sum dOut y) / (n mu),   dweight = sum_rows dOut x / mu
    sign(0) = 0 as torch.abs differentiates it."""
    n = x.shape[-1]
    mu = x.abs().mean(-1, keepdim=True) + eps
    xn = x / mu
    c = (d_out * xn * weight).sum(-1, keepdim=True)
    dx = d_out * weight / mu - torch.sign(x) * c / (n * mu)
    dw = (d_out * xn).reshape(-1, n).sum(0)
    return dx, dw


def autograd_grads(fn, inputs, d_out):
    """Gradients of ``fn(*inputs)`` w.r.t. every input, through torch autograd."""
    leaves = [t.detach().clone().requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    out.backward(d_out)
    return out.detach(), [t.grad for t in leaves]


# --------------------------------------------------------------------------------------
# the language model (algebraic_model.py:26-237), as a pure function of a state dict
# --------------------------------------------------------------------------------------

def lm_forward(state: Dict[str, torch.Tensor], input_ids: torch.Tensor, n_head: int,
               labels: Optional[torch.Tensor] = None,
               attention_mask: Optional[torch.Tensor] = None,
               eps: float = EPS) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Forward pass of AlgebraicTransformerLM with dropout 0, keyed like its state_dict:
    ``head.weight`` (tied to the embedding, algebraic_model.py:193), ``blocks.{i}.norm1.weight``,
    ``blocks.{i}.attn.qkv.weight``, ``blocks.{i}.attn.out.weight``, ``blocks.{i}.norm2.weight``,
    ``blocks.{i}.ffn.w_gate_val.weight``, ``blocks.{i}.ffn.w_out.weight``, ``norm.weight``.
    Returns (logits, loss); loss is the shifted cross entropy (algebraic_model.py:229-235)."""
    emb = state["head.weight"]
    x = emb[input_ids]
    B, T, C = x.shape
    d_head = C // n_head
    slopes = compute_alibi_slopes(n_head)
    n_layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("blocks."))
    for i in range(n_layers):
        pre = f"blocks.{i}."
        h = mean_error_norm(x, state[pre + "norm1.weight"], eps)
        qkv = (h @ state[pre + "attn.qkv.weight"].t()).view(B, T, 3, n_head, d_head)
        q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
        s = _scores(q, k, slopes, 1.0 / math.sqrt(d_head))
        if attention_mask is not None:      # padding mask, CPU path only (algebraic_model.py:128-131)
            s = s.masked_fill(attention_mask[:, None, None, :] == 0, MASK_FILL)
        a = torch.matmul(rational_softmax(s, eps), v)
        x = x + a.transpose(1, 2).reshape(B, T, C) @ state[pre + "attn.out.weight"].t()
        h = mean_error_norm(x, state[pre + "norm2.weight"], eps)
        gate, val = (h @ state[pre + "ffn.w_gate_val.weight"].t()).chunk(2, dim=-1)
        x = x + rational_swiglu(gate, val) @ state[pre + "ffn.w_out.weight"].t()
    logits = mean_error_norm(x, state["norm.weight"], eps) @ emb.t()
    loss = None
    if labels is not None:
        loss = torch.nn.functional.cross_entropy(
            logits[:, :-1].reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
            ignore_index=-100)
    return logits, loss


def lm_loss_and_grads(state, input_ids, labels, n_head):
    """(loss, {name: grad}) for the pure-function model above, via autograd."""
    leaves = {k: v.detach().clone().float().requires_grad_(True) for k, v in state.items()}
    _, loss = lm_forward(leaves, input_ids, n_head, labels)
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in leaves.items()}
