"""AlgebraicTransformerLM on the CUDA operators against the golden vectors and the CPU oracle (B200)."""
import pytest
import torch

from conftest import load_golden, norm_max_err
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build_from_golden(dtype=torch.float32, **kw):
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM
    g = load_golden("lm_tiny")
    model = AlgebraicTransformerLM(vocab_size=128, d_model=64, n_head=int(g["n_head"]), n_layers=2, dropout=0.0, **kw)
    state = {k[3:].replace("__", "."): v for k, v in g.items() if k.startswith("w__")}
    missing, unexpected = model.load_state_dict(state, strict=False)
    assert not unexpected and set(missing) <= {"head.weight"} | {f"blocks.{i}.attn.alibi_slopes" for i in range(2)}
    return model.to(DEV).to(dtype).train(), g


def test_lm_tiny_matches_reference_golden():
    model, g = build_from_golden()
    logits, loss = model(g["input_ids"].to(DEV), labels=g["labels"].to(DEV))
    assert norm_max_err(logits, g["logits"]) < 1e-5
    assert abs(loss.item() - g["loss"]) < 1e-5
    loss.backward()
    for name, p in model.named_parameters():
        assert norm_max_err(p.grad, g["g__" + name.replace(".", "__")]) < 5e-5, name


def test_lm_gradient_checkpointing_gives_same_gradients():
    model, g = build_from_golden(gradient_checkpointing=True)
    _, loss = model(g["input_ids"].to(DEV), labels=g["labels"].to(DEV))
    loss.backward()
    for name, p in model.named_parameters():
        assert norm_max_err(p.grad, g["g__" + name.replace(".", "__")]) < 5e-5, name


def test_lm_state_dict_names_match_reference():
    model, g = build_from_golden()
    ref_names = {k[3:].replace("__", ".") for k in g if k.startswith("w__")}
    assert {n for n, _ in model.named_parameters()} == ref_names


def test_lm_bf16_close_to_fp32_oracle():
    """A bf16 step of a mid-sized model (D=64 heads, tensor-core attention) stays close to the fp32 oracle."""
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM
    torch.manual_seed(31)
    model = AlgebraicTransformerLM(vocab_size=512, d_model=256, n_head=4, n_layers=2, dropout=0.0)
    ids = torch.randint(0, 512, (2, 192)); labels = torch.randint(0, 512, (2, 192))
    state = {k: v.detach().clone() for k, v in model.state_dict().items()
             if k != "embed.weight" and not k.endswith("alibi_slopes")}
    state = {k: v.to(torch.bfloat16).float() for k, v in state.items()}
    want_loss, want_grads = oracle.lm_loss_and_grads(state, ids, labels, 4)
    model = model.to(DEV).to(torch.bfloat16).train()
    _, loss = model(ids.to(DEV), labels=labels.to(DEV))
    loss.backward()
    assert abs(loss.item() - want_loss.item()) < 2e-2
    got = model.blocks[0].attn.qkv.weight.grad.float()
    assert norm_max_err(got, want_grads["blocks.0.attn.qkv.weight"]) < 5e-2


def test_generate_runs():
    model, g = build_from_golden()
    model.eval()
    out = model.generate(g["input_ids"][:1, :8].to(DEV), max_new_tokens=4, top_k=5)
    assert out.shape == (1, 12)


def test_lm_without_logits_gives_the_same_loss_and_gradients():
    """return_logits=False: the head GEMM and the loss run one sequence at a time, the [B, T, V] logits never exist.
    Same loss and parameter gradients as the reference's golden vectors."""
    model, g = build_from_golden()
    logits, loss = model(g["input_ids"].to(DEV), labels=g["labels"].to(DEV), return_logits=False)
    assert logits is None
    assert abs(loss.item() - g["loss"]) < 1e-5
    loss.backward()
    for name, p in model.named_parameters():
        assert norm_max_err(p.grad, g["g__" + name.replace(".", "__")]) < 5e-5, name
    with pytest.raises(ValueError):
        model(g["input_ids"].to(DEV), return_logits=False)


def test_loss_backward_twice_is_refused_not_wrong():
    """The loss gradients are scaled in place in the backward; a second backward over the same graph would scale them
    twice, so it raises instead."""
    model, g = build_from_golden()
    for keep in (True, False):
        _, loss = model(g["input_ids"].to(DEV), labels=g["labels"].to(DEV), return_logits=keep)
        loss.backward(retain_graph=True)
        with pytest.raises(RuntimeError, match="twice"):
            loss.backward()
        model.zero_grad(set_to_none=True)
