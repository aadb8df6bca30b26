"""Algebraic Transformer language model on the sm_100a operators.

Host-side mirror of the reference's ``algebraic_model.py`` (RationalMR 26-39, RationalSwiGLU
42-62, AlgebraicAttention 65-136, AlgebraicBlock 139-152, AlgebraicTransformerLM 155-265,
factories 272-302): same module names, constructor arguments, parameter names (so state
dicts are interchangeable) and forward signature.  The modules run on CUDA only.

Differences that remove copies but not behaviour: q, k, v are handed to the attention kernels
as strided views of the packed projection, the attention output is produced directly in
[B, T, H*D] memory order, and the SwiGLU kernels read the gate/value halves in place.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from . import ops
from .backward import RationalAttentionPackedFunction
from .forward import compute_alibi_slopes
from .fused_ops import (EPS, RationalSwiGLUPacked, add_mean_error_norm, head_shifted_cross_entropy, mean_error_norm,
                        shifted_cross_entropy)


class RationalMR(nn.Module):
    """Mean-error normalisation layer (reference algebraic_model.py:26-39)."""

    def __init__(self, d_model: int, eps: float = EPS):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d_model))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return mean_error_norm(x, self.weight, self.eps)


class RationalSwiGLU(nn.Module):
    """SwiGLU feed-forward block with the rational sigmoid (reference algebraic_model.py:42-62)."""

    def __init__(self, d_model: int, d_ffn: int, dropout: float = 0.0):
        super().__init__()
        self.w_gate_val = nn.Linear(d_model, 2 * d_ffn, bias=False)
        self.w_out = nn.Linear(d_ffn, d_model, bias=False)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gv = self.w_gate_val(x)
        if not gv.is_cuda:
            raise RuntimeError("RationalSwiGLU: CUDA tensor required — this build has no CPU fallback")
        return self.dropout(self.w_out(RationalSwiGLUPacked.apply(gv)))


class KVCache:
    """Keys and values of the tokens a model has seen, for ``generate``: one [B, H, capacity, D] pair per layer and the
    number of cached tokens per sequence as an int32 tensor on the device (the decode kernel reads it there, so a step
    looks the same to the GPU whatever the length).  The reference has no cache: its generate() runs the whole prefix
    through forward() for every new token (algebraic_model.py:239-265)."""

    DECODE_HEAD_SIZES = (32, 64, 128)
    DECODE_DTYPES = (torch.float32, torch.bfloat16, torch.float16)

    def __init__(self, n_layers: int, batch: int, n_head: int, capacity: int, d_head: int, dtype: torch.dtype, device):
        self.capacity = capacity
        self.k = [torch.empty(batch, n_head, capacity, d_head, dtype=dtype, device=device) for _ in range(n_layers)]
        self.v = [torch.empty(batch, n_head, capacity, d_head, dtype=dtype, device=device) for _ in range(n_layers)]
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=device)
        self.seen = 0                                   # host copy of the (common) length

    def layer(self, i: int):
        return self.k[i], self.v[i], self

    def advance(self, n_tokens: int) -> None:
        """Called once per model step, after every layer has appended its rows."""
        self.lengths += n_tokens
        self.seen += n_tokens


class AlgebraicAttention(nn.Module):
    """Multi-head causal attention with rational softmax and ALiBi (reference algebraic_model.py:65-110).

    ``mask`` [B, T] (0 = padding) takes the padded keys out of every query's sum, as the reference's PyTorch path does
    (algebraic_model.py:128-131: their scores are filled with -1e4); the reference's Triton path drops the argument
    (algebraic_model.py:93-104), so on CUDA this is where the two differ: here the mask counts."""

    def __init__(self, d_model: int, n_head: int, dropout: float = 0.1):
        super().__init__()
        assert d_model % n_head == 0
        self.d_model = d_model
        self.n_head = n_head
        self.d_head = d_model // n_head
        self.scale = 1.0 / math.sqrt(self.d_head)
        self.qkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.out = nn.Linear(d_model, d_model, bias=False)
        self.dropout = nn.Dropout(dropout)
        self.register_buffer("alibi_slopes", compute_alibi_slopes(n_head))

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None, cache=None) -> torch.Tensor:
        """``cache`` (an extension): ``KVCache.layer(i)``.  An empty cache is filled with this call's keys and values (the
        prompt); afterwards ``x`` must hold one new token per sequence, which is appended and attends over the cache."""
        B, T, C = x.shape
        qkv = self.qkv(x).view(B, T, 3, self.n_head, self.d_head)
        if not qkv.is_cuda:
            raise RuntimeError("AlgebraicAttention: CUDA tensor required — this build has no CPU fallback")
        if cache is not None and cache[2].seen > 0:
            k_cache, v_cache, state = cache
            if T != 1:
                raise ValueError("a filled key/value cache takes one new token per sequence and step")
            if state.seen >= state.capacity:
                raise RuntimeError(f"key/value cache is full ({state.capacity} tokens)")
            out = ops.attn_decode(qkv[:, 0, 0], qkv[:, 0, 1], qkv[:, 0, 2], k_cache, v_cache, state.lengths, self.alibi_slopes,
                                  float(self.scale), float(EPS)).view(B, 1, C)
            return self.dropout(self.out(out))
        if mask is not None and cache is not None:
            raise ValueError("the key/value cache takes no padding mask")
        out = RationalAttentionPackedFunction.apply(qkv, self.alibi_slopes, self.scale, EPS, mask)     # [B,T,C]
        if cache is not None:
            k_cache, v_cache, state = cache
            if T > state.capacity:
                raise RuntimeError(f"the prompt ({T} tokens) does not fit the key/value cache ({state.capacity})")
            k_cache[:, :, :T].copy_(qkv[:, :, 1].permute(0, 2, 1, 3))
            v_cache[:, :, :T].copy_(qkv[:, :, 2].permute(0, 2, 1, 3))
        return self.dropout(self.out(out))


class AlgebraicBlock(nn.Module):
    """Pre-norm transformer block (reference algebraic_model.py:139-152)."""

    def __init__(self, d_model: int, n_head: int, d_ffn: int, dropout: float):
        super().__init__()
        self.attn = AlgebraicAttention(d_model, n_head, dropout)
        self.ffn = RationalSwiGLU(d_model, d_ffn, dropout)
        self.norm1 = RationalMR(d_model)
        self.norm2 = RationalMR(d_model)

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None, cache=None) -> torch.Tensor:
        x = x + self.attn(self.norm1(x), mask, cache)
        return x + self.ffn(self.norm2(x))

    def forward_deferred(self, x: torch.Tensor, pending: Optional[torch.Tensor],
                         mask: Optional[torch.Tensor] = None, cache=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """The same block with every residual addition fused into the normalisation that follows it.  ``pending`` is
        the previous block's feed-forward output that has not been added to ``x`` yet (None for the first block);
        returns (x, pending) in the same convention: the caller adds the last pending term (or fuses it into the
        final norm).  Same numbers as ``forward``: the sums are rounded to the tensor dtype before they are normalised."""
        if pending is None:
            y = self.norm1(x)
        else:
            x, y = add_mean_error_norm(x, pending, self.norm1.weight, self.norm1.eps)
        x, y = add_mean_error_norm(x, self.attn(y, mask, cache), self.norm2.weight, self.norm2.eps)
        return x, self.ffn(y)


class AlgebraicTransformerLM(nn.Module):
    """Algebraic Transformer language model (reference algebraic_model.py:155-265)."""

    def __init__(self, vocab_size: int, d_model: int, n_head: int, n_layers: int, d_ffn: Optional[int] = None,
                 block_size: int = 2048, dropout: float = 0.1, gradient_checkpointing: bool = False, **kwargs):
        super().__init__()
        if d_ffn is None:
            d_ffn = int(d_model * 8 / 3)
        self.block_size = block_size
        self.gradient_checkpointing = gradient_checkpointing
        self.n_layers = n_layers
        self.embed = nn.Embedding(vocab_size, d_model)
        self.blocks = nn.ModuleList([AlgebraicBlock(d_model, n_head, d_ffn, dropout) for _ in range(n_layers)])
        self.norm = RationalMR(d_model)
        self.head = nn.Linear(d_model, vocab_size, bias=False)
        self.embed.weight = self.head.weight            # tied (reference algebraic_model.py:193)
        self.apply(self._init_weights)

    def _init_weights(self, module):
        if isinstance(module, nn.Linear):
            std = 0.02
            if hasattr(module, "_scale_init"):
                std = 0.02 / math.sqrt(2 * self.n_layers)
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None,
                return_logits: bool = True) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """(logits, loss) as the reference returns them (algebraic_model.py:209-237).  ``return_logits=False`` (an
        extension; needs ``labels``) is for training loops that only use the loss: the head GEMM and the loss then run one
        sequence at a time and neither the [B, T, V] logits nor their gradient are ever materialised; ``logits`` is None."""
        x = self.embed(input_ids)
        if attention_mask is not None and not isinstance(attention_mask, ops.PackedKeyMask):
            attention_mask = ops.PackedKeyMask(attention_mask)          # packed to bits once for all layers
        if self.gradient_checkpointing and self.training:
            for block in self.blocks:
                x = checkpoint(block, x, attention_mask, use_reentrant=False)
            y = self.norm(x)
        else:
            # residual additions travel with the next normalisation (one pass instead of two per sublayer)
            pending = None
            for block in self.blocks:
                x, pending = block.forward_deferred(x, pending, attention_mask)
            if pending is None:
                y = self.norm(x)
            else:
                _, y = add_mean_error_norm(x, pending, self.norm.weight, self.norm.eps)
        if not return_logits:
            if labels is None:
                raise ValueError("return_logits=False needs labels (there would be nothing to return)")
            if y.dim() == 3 and y.dtype in (torch.float32, torch.bfloat16, torch.float16):
                return None, head_shifted_cross_entropy(y, self.head.weight, labels, -100)
        logits = self.head(y)
        loss = None
        if labels is not None:
            if logits.dim() == 3 and logits.dtype in (torch.float32, torch.bfloat16, torch.float16):
                # one pass over the logits yields the loss and its gradient (no shifted copy, no log-softmax tensor)
                loss = shifted_cross_entropy(logits, labels, -100)
            else:
                shift_logits = logits[..., :-1, :].contiguous()
                shift_labels = labels[..., 1:].contiguous()
                loss = F.cross_entropy(shift_logits.view(-1, shift_logits.size(-1)), shift_labels.view(-1),
                                       ignore_index=-100)
        return (logits if return_logits else None), loss

    def new_cache(self, batch: int, capacity: int) -> KVCache:
        """An empty key/value cache for ``batch`` sequences of up to ``capacity`` tokens, in the model's dtype and device."""
        attn = self.blocks[0].attn
        w = self.head.weight
        return KVCache(len(self.blocks), batch, attn.n_head, capacity, attn.d_head, w.dtype, w.device)

    def cache_supported(self) -> bool:
        """Whether the decode kernel covers this model's head size and dtype (else ``generate`` recomputes the prefix)."""
        w = self.head.weight
        return w.is_cuda and self.blocks[0].attn.d_head in KVCache.DECODE_HEAD_SIZES and w.dtype in KVCache.DECODE_DTYPES

    @torch.no_grad()
    def forward_cached(self, input_ids: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """Logits [B, V] of the LAST position of ``input_ids`` given the tokens already in ``cache``.  With an empty cache
        ``input_ids`` is the prompt (any length); afterwards it is the one token per sequence that was sampled last.
        Same arithmetic as ``forward`` on the concatenated sequence: keys and values of earlier positions do not
        depend on later tokens (causal attention, relative bias), so they are kept instead of recomputed."""
        x = self.embed(input_ids)
        pending = None
        for i, block in enumerate(self.blocks):
            x, pending = block.forward_deferred(x, pending, None, cache.layer(i))
        x, pending = x[:, -1:], pending[:, -1:]
        _, y = add_mean_error_norm(x.contiguous(), pending.contiguous(), self.norm.weight, self.norm.eps)
        cache.advance(input_ids.size(1))
        return self.head(y)[:, -1, :]

    @torch.no_grad()
    def generate(self, idx: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, use_cache: bool = True, cuda_graph: bool = True) -> torch.Tensor:
        """Sampling loop (reference algebraic_model.py:239-265).  The reference re-runs the forward over the whole prefix
        for every token; here (``use_cache``, an extension) the prompt runs once, its keys and values are kept, and each
        new token costs one decode step.  The two agree as long as the reference would not crop the prefix to
        ``block_size``; when it would (or the decode kernel does not cover the model), the reference's loop runs.
        ``cuda_graph``: a decode step is a hundred small launches whatever the length (the cached lengths live on the
        device), so after one step issued launch by launch it is captured once and replayed for the remaining tokens."""
        def sample(logits):
            if temperature != 1.0:
                logits = logits / temperature
            if top_k is not None:
                kth, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < kth[:, [-1]]] = float("-inf")
            return torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)

        longest = idx.size(1) + max_new_tokens - 1          # the longest prefix a forward pass will see
        if use_cache and max_new_tokens > 0 and idx.size(1) > 0 and longest <= self.block_size and self.cache_supported():
            cache = self.new_cache(idx.size(0), longest)
            logits = self.forward_cached(idx, cache)
            graph = token = None
            for step in range(max_new_tokens):
                nxt = sample(logits)
                idx = torch.cat((idx, nxt), dim=1)
                if step + 1 == max_new_tokens:
                    break
                if graph is not None:
                    token.copy_(nxt)
                    graph.replay()
                    cache.seen += 1                         # (the device-side lengths advance inside the graph)
                elif cuda_graph and step == 1 and max_new_tokens - step > 4:
                    token, seen = nxt.clone(), cache.seen
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        logits = self.forward_cached(token, cache)
                    cache.seen = seen                       # capturing ran the host bookkeeping without running the step
                    graph.replay()
                    cache.seen += 1
                else:
                    logits = self.forward_cached(nxt, cache)
            return idx
        for _ in range(max_new_tokens):
            idx_cond = idx if idx.size(1) <= self.block_size else idx[:, -self.block_size:]
            logits, _ = self.forward(idx_cond)
            idx = torch.cat((idx, sample(logits[:, -1, :])), dim=1)
        return idx


def create_small_model(vocab_size: int = 32000, **kwargs) -> AlgebraicTransformerLM:
    """~125M parameters (reference algebraic_model.py:272-280)."""
    return AlgebraicTransformerLM(vocab_size=vocab_size, d_model=768, n_head=12, n_layers=12, **kwargs)


def create_medium_model(vocab_size: int = 32000, **kwargs) -> AlgebraicTransformerLM:
    """~350M parameters (reference algebraic_model.py:283-291)."""
    return AlgebraicTransformerLM(vocab_size=vocab_size, d_model=1024, n_head=16, n_layers=24, **kwargs)


def create_large_model(vocab_size: int = 32000, **kwargs) -> AlgebraicTransformerLM:
    """~760M parameters (reference algebraic_model.py:294-302)."""
    return AlgebraicTransformerLM(vocab_size=vocab_size, d_model=1536, n_head=24, n_layers=24, **kwargs)


def create_xl_model(vocab_size: int = 50000, **kwargs) -> AlgebraicTransformerLM:
    """~1.3B parameters: d_model 2048, 16 heads, 24 layers, FFN hidden 5504 (the reference's README
    advertises this factory without defining it)."""
    kwargs.setdefault("d_ffn", 5504)
    return AlgebraicTransformerLM(vocab_size=vocab_size, d_model=2048, n_head=16, n_layers=24, **kwargs)
