"""Decode step over a key/value cache (fat_attn_decode) and the cached ``generate`` (B200).

The reference has no cache: its generate() re-runs forward() over the whole prefix for every token
(algebraic_model.py:239-265).  The pin is therefore the causal attention itself: the decode step of the token at position
n must equal row n of the oracle's causal attention over the n+1 tokens, and the cached model must give the logits the
full forward gives at the same position.
"""
import ctypes

import pytest
import torch

from conftest import bf16_violations, norm_max_err
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(dtype, B, H, D, capacity, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, D, generator=g).to(dtype)
    k_new = torch.randn(B, H, D, generator=g).to(dtype)
    v_new = torch.randn(B, H, D, generator=g).to(dtype)
    kc = torch.randn(B, H, capacity, D, generator=g).to(dtype)
    vc = torch.randn(B, H, capacity, D, generator=g).to(dtype)
    for b, n in enumerate(lengths):                 # rows that are not part of the sequence must never be read
        kc[b, :, n:] = float("nan")
        vc[b, :, n:] = float("nan")
    return q, k_new, v_new, kc, vc


def _oracle_rows(q, k_new, v_new, kc, vc, lengths, slopes, scale):
    rows = []
    for b, n in enumerate(lengths):
        k = torch.cat((kc[b, :, :n].float(), k_new[b].float()[:, None]), 1)[None]        # [1,H,n+1,D]
        v = torch.cat((vc[b, :, :n].float(), v_new[b].float()[:, None]), 1)[None]
        rows.append(oracle.rational_attention_last_row(q[b].float()[None], k, v, slopes, scale)[0])
    return torch.stack(rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,D,capacity,lengths", [
    (2, 4, 64, 300, (0, 299)),                      # an empty cache and one that the new row fills
    (3, 12, 64, 1024, (17, 511, 1000)),             # the small model's heads (non-power-of-two slopes)
    (2, 2, 128, 4096, (4095, 2500)),                # few (batch, head) pairs: the key range is split over 8 CTAs
    (1, 16, 128, 2048, (1234,)),                    # the XL model's heads
    (2, 3, 32, 96, (5, 64)),
])
def test_decode_step_equals_last_row_of_causal_attention(dtype, B, H, D, capacity, lengths):
    from fastalgebraictransformer_b200 import ops
    slopes = oracle.compute_alibi_slopes(H)
    scale = D ** -0.5
    q, k_new, v_new, kc, vc = _case(dtype, B, H, D, capacity, lengths, 7 + D + B)
    want = _oracle_rows(q, k_new, v_new, kc, vc, lengths, slopes, scale)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    n_cached = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    got = ops.attn_decode(q.to(DEV), k_new.to(DEV), v_new.to(DEV), kc_d, vc_d, n_cached, slopes.to(DEV), scale, 1e-6)
    if dtype == torch.float32:
        assert norm_max_err(got, want) < 1e-5
    else:
        bad, _ = bf16_violations(got, want)
        assert bad == 0.0                            # every element inside |a-b| <= 1e-2 + 2e-2|b|
    for b, n in enumerate(lengths):                  # the new rows were appended, nothing else moved
        assert torch.equal(kc_d[b, :, n].cpu(), k_new[b]) and torch.equal(vc_d[b, :, n].cpu(), v_new[b])
        assert torch.equal(kc_d[b, :, :n].cpu(), kc[b, :, :n]) and torch.equal(vc_d[b, :, :n].cpu(), vc[b, :, :n])
        assert torch.isnan(kc_d[b, :, n + 1:]).all() and torch.isnan(vc_d[b, :, n + 1:]).all()
    # same arguments, same bits
    kc2, vc2 = kc.to(DEV), vc.to(DEV)
    again = ops.attn_decode(q.to(DEV), k_new.to(DEV), v_new.to(DEV), kc2, vc2, n_cached, slopes.to(DEV), scale, 1e-6)
    assert torch.equal(got, again)


def test_decode_reads_strided_views_of_the_packed_projection():
    """q, k_new, v_new as the model passes them: slices of one [B, 1, 3, H, D] projection output."""
    from fastalgebraictransformer_b200 import ops
    B, H, D, cap, n = 2, 4, 64, 128, 40
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, 1, 3, H, D, generator=g).to(torch.bfloat16)
    kc = torch.randn(B, H, cap, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(B, H, cap, D, generator=g).to(torch.bfloat16)
    slopes = oracle.compute_alibi_slopes(H)
    want = _oracle_rows(qkv[:, 0, 0], qkv[:, 0, 1], qkv[:, 0, 2], kc, vc, (n, n), slopes, 0.125)
    qkv_d = qkv.to(DEV)
    got = ops.attn_decode(qkv_d[:, 0, 0], qkv_d[:, 0, 1], qkv_d[:, 0, 2], kc.to(DEV), vc.to(DEV),
                          torch.full((B,), n, dtype=torch.int32, device=DEV), slopes.to(DEV), 0.125, 1e-6)
    assert bf16_violations(got, want)[0] == 0.0


def test_decode_reports_a_full_cache_through_the_c_abi():
    """A sequence whose cache has no room gets zeros, nothing is written, and the status word says so."""
    from fastalgebraictransformer_b200 import _lib
    lib = _lib.lib()
    B, H, D, cap = 2, 2, 64, 16
    q = torch.randn(B, H, D, device=DEV)
    kc = torch.randn(B, H, cap, D, device=DEV)
    vc = torch.randn(B, H, cap, D, device=DEV)
    kc0, vc0 = kc.clone(), vc.clone()
    out = torch.full((B, H, D), 7.0, device=DEV)
    n_cached = torch.tensor([3, cap], dtype=torch.int32, device=DEV)      # the second sequence is full
    slopes = oracle.compute_alibi_slopes(H).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    s2 = (ctypes.c_int64 * 2)(H * D, D)
    s3 = (ctypes.c_int64 * 3)(H * cap * D, cap * D, D)
    rc = lib.fat_attn_decode(q.data_ptr(), q.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), n_cached.data_ptr(),
                             slopes.data_ptr(), out.data_ptr(), B, H, cap, D, s2, s2, s2, s2, s3, s3, 0.125, 1e-6, _lib.F32,
                             status.data_ptr(), _lib.stream_ptr(q.device))
    assert rc == 0, lib.fat_last_error().decode()
    torch.cuda.synchronize()
    assert status.item() == 0x10000000
    assert torch.all(out[1] == 0) and torch.isfinite(out[0]).all() and not torch.all(out[0] == 0)
    assert torch.equal(kc[1], kc0[1]) and torch.equal(vc[1], vc0[1])
    assert torch.equal(kc[0, :, 3], q[0])                                 # the other sequence was served normally
    # refused on the host: a head size without a kernel, misaligned rows
    rc = lib.fat_attn_decode(q.data_ptr(), q.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), n_cached.data_ptr(),
                             slopes.data_ptr(), out.data_ptr(), B, H, cap, 48, s2, s2, s2, s2, s3, s3, 0.125, 1e-6, _lib.F32,
                             status.data_ptr(), None)
    assert rc == 3
    rc = lib.fat_attn_decode(q.data_ptr() + 4, q.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), n_cached.data_ptr(),
                             slopes.data_ptr(), out.data_ptr(), B, H, cap, D, s2, s2, s2, s2, s3, s3, 0.125, 1e-6, _lib.F32,
                             status.data_ptr(), None)
    assert rc == 4


def _tiny(dtype, d_model=64, n_head=2, n_layers=2, vocab=128, block_size=64):
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM
    torch.manual_seed(11)
    model = AlgebraicTransformerLM(vocab_size=vocab, d_model=d_model, n_head=n_head, n_layers=n_layers, dropout=0.0,
                                   block_size=block_size)
    return model.to(DEV).to(dtype).eval()


@pytest.mark.parametrize("dtype,d_model,n_head", [(torch.float32, 64, 2), (torch.bfloat16, 256, 4), (torch.bfloat16, 256, 2)])
def test_cached_steps_give_the_logits_of_the_full_forward(dtype, d_model, n_head):
    """Prompt of 20 tokens, then 12 tokens one at a time: at every step the cached logits are the full forward's."""
    from fastalgebraictransformer_b200 import AlgebraicTransformerLM
    torch.manual_seed(11)
    model = AlgebraicTransformerLM(vocab_size=512, d_model=d_model, n_head=n_head, n_layers=2, dropout=0.0, block_size=64)
    ids = torch.randint(0, 512, (3, 32))
    # the pin: the reference's forward as the oracle restates it, in float32 on the (rounded) weights
    state = {k: v.detach().to(dtype).float() for k, v in model.state_dict().items()
             if k != "embed.weight" and not k.endswith("alibi_slopes")}
    want, _ = oracle.lm_forward(state, ids, n_head)
    model = model.to(DEV).to(dtype).eval()
    ids = ids.to(DEV)
    with torch.no_grad():
        full, _ = model(ids)
        cache = model.new_cache(3, 32)
        got = [model.forward_cached(ids[:, :20], cache)]
        for t in range(20, 32):
            got.append(model.forward_cached(ids[:, t:t + 1], cache))
    assert cache.seen == 32 and cache.lengths.tolist() == [32, 32, 32]
    # float32: the bar of the other float32 tests.  bfloat16: two layers of 16-bit operators and GEMMs in a row; the cached
    # steps must be as close to the float32 oracle as the full forward is (normalised error, like the model-level 16-bit test)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert norm_max_err(full[:, 19:], want[:, 19:]) < tol
    for i, t in enumerate(range(19, 32)):
        assert norm_max_err(got[i], want[:, t]) < tol, t
        if dtype == torch.float32:
            assert norm_max_err(got[i], full[:, t]) < 1e-5, t


def test_generate_with_cache_equals_the_reference_loop():
    """Greedy sampling (top_k=1 leaves one candidate) through the cache and through the reference's recompute loop."""
    model = _tiny(torch.float32, block_size=48)
    prompt = torch.randint(0, 128, (2, 9), device=DEV)
    a = model.generate(prompt.clone(), 24, top_k=1, use_cache=True)                      # decode steps replayed from a CUDA graph
    b = model.generate(prompt.clone(), 24, top_k=1, use_cache=False)
    e = model.generate(prompt.clone(), 24, top_k=1, use_cache=True, cuda_graph=False)    # every decode step launch by launch
    assert a.shape == (2, 33) and torch.equal(a, b) and torch.equal(e, b)
    fat_status = __import__("fastalgebraictransformer_b200").check_device_status
    fat_status()                                                                         # no cache overflow was reported
    # a run that would outgrow block_size falls back to the reference's loop (the window slides, positions shift)
    c = model.generate(prompt.clone(), 48, top_k=1, use_cache=True)
    d = model.generate(prompt.clone(), 48, top_k=1, use_cache=False)
    assert c.shape == (2, 57) and torch.equal(c, d)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_decode_first_token_of_an_empty_cache(dtype):
    """n_cached = 0 everywhere and a cache of one row: the token attends to itself only, out = v * f / (f + eps)."""
    from fastalgebraictransformer_b200 import ops
    B, H, D = 2, 3, 32
    g = torch.Generator().manual_seed(2)
    q, k_new, v_new = (torch.randn(B, H, D, generator=g).to(dtype) for _ in range(3))
    kc = torch.full((B, H, 1, D), float("nan"), dtype=dtype)
    vc = torch.full((B, H, 1, D), float("nan"), dtype=dtype)
    slopes = oracle.compute_alibi_slopes(H)
    want = oracle.rational_attention_last_row(q.float(), k_new.float()[:, :, None], v_new.float()[:, :, None], slopes, 0.2)
    kd, vd = kc.to(DEV), vc.to(DEV)
    got = ops.attn_decode(q.to(DEV), k_new.to(DEV), v_new.to(DEV), kd, vd, torch.zeros(B, dtype=torch.int32, device=DEV),
                          slopes.to(DEV), 0.2, 1e-6)
    if dtype == torch.float32:
        assert norm_max_err(got, want) < 1e-5
    else:
        assert bf16_violations(got, want)[0] == 0.0
    assert torch.equal(kd[:, :, 0].cpu(), k_new) and torch.equal(vd[:, :, 0].cpu(), v_new)
