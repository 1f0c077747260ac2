"""Flash attention kernels vs an fp32 softmax(QK^T)V reference (GQA, MHA, MLA shapes; causal and full)."""
import math

import pytest
import torch

from primus_b200.ops import _lib
from primus_b200.ops import attention as A

pytestmark = pytest.mark.gpu

CASES = [
    # batch, seq, hq, hkv, dqk, dv, causal
    (1, 128, 2, 2, 128, 128, True),
    (1, 512, 4, 2, 128, 128, True),
    (2, 384, 4, 1, 128, 128, True),
    (1, 256, 2, 2, 128, 128, False),
    (1, 512, 4, 2, 64, 64, True),
    (1, 384, 2, 2, 192, 128, True),
]


def _inputs(batch, seq, hq, hkv, dqk, dv, packed=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = batch * seq
    if packed and dqk == dv:
        qkv = torch.randn(T, (hq + 2 * hkv) * dqk, device="cuda", generator=g).bfloat16()
        q = qkv[:, : hq * dqk].view(T, hq, dqk)
        k = qkv[:, hq * dqk: (hq + hkv) * dqk].view(T, hkv, dqk)
        v = qkv[:, (hq + hkv) * dqk:].view(T, hkv, dv)
        return q, k, v
    q = torch.randn(T, hq, dqk, device="cuda", generator=g).bfloat16()
    k = torch.randn(T, hkv, dqk, device="cuda", generator=g).bfloat16()
    v = torch.randn(T, hkv, dv, device="cuda", generator=g).bfloat16()
    return q, k, v


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("packed", [False, True])
def test_flash_attn_forward(case, packed):
    batch, seq, hq, hkv, dqk, dv, causal = case
    q, k, v = _inputs(batch, seq, hq, hkv, dqk, dv, packed)
    scale = 1.0 / math.sqrt(dqk)
    o, lse = A.flash_attn_fwd(q, k, v, batch, causal, scale)
    torch.cuda.synchronize()
    _lib.check_status()
    o_ref, lse_ref = A.attention_ref(q, k, v, batch, causal, scale)
    assert (o.float() - o_ref.float()).abs().max().item() <= 2e-2
    assert (lse - lse_ref).abs().max().item() <= 2e-2


@pytest.mark.parametrize("case", CASES)
def test_flash_attn_backward(case):
    batch, seq, hq, hkv, dqk, dv, causal = case
    q, k, v = _inputs(batch, seq, hq, hkv, dqk, dv, seed=1)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = A.flash_attention(q, k, v, batch, causal)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = A.attention_ref(qr, kr, vr, batch, causal)
    o_ref.backward(do.float())
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 3e-2 * b.abs().max().item() + 2e-2
        assert err <= tol, f"{name}: err {err} tol {tol}"


def test_flash_attn_fwd_bwd_at_the_benchmark_length():
    """seq 8192 (64 key blocks, many waves of streamed tiles per CTA), one GQA group of the Llama-3.1-8B shape
    (4 query heads on 1 KV head, d 128), forward and backward against the fp32 reference."""
    batch, seq, hq, hkv, d = 1, 8192, 4, 1, 128
    q, k, v = _inputs(batch, seq, hq, hkv, d, d, seed=7)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = A.flash_attention(q, k, v, batch, True)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = A.attention_ref(qr, kr, vr, batch, True)
    o_ref.backward(do.float())
    assert (o.float() - o_ref.float()).abs().max().item() <= 2e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 3e-2 * b.abs().max().item() + 2e-2
        assert err <= tol, f"{name}: err {err} tol {tol}"
        rel = (a.float() - b).norm().item() / b.norm().item()
        assert rel <= 1e-2, f"{name}: relative error {rel}"


def test_flash_attn_deterministic():
    q, k, v = _inputs(1, 1024, 8, 2, 128, 128, seed=3)
    o1, l1 = A.flash_attn_fwd(q, k, v, 1, True, 0.088)
    o2, l2 = A.flash_attn_fwd(q, k, v, 1, True, 0.088)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


CHUNK_CASES = [
    # batch, seq_q, q_off, hq, hkv, dqk, dv, causal
    (1, 128, 128, 2, 2, 128, 128, True),
    (1, 256, 384, 4, 2, 128, 128, True),
    (2, 128, 256, 4, 1, 128, 128, True),
    (1, 384, 0, 2, 2, 128, 128, True),
    (1, 256, 256, 2, 2, 192, 128, True),
    (1, 128, 0, 2, 2, 128, 128, False),     # cross attention: 128 queries over 384 keys
]


@pytest.mark.parametrize("case", CHUNK_CASES)
def test_flash_attn_chunk_against_longer_keys(case):
    """Queries of a sequence chunk at key position q_off attending to keys [0, q_off + seq_q) (forward and backward)."""
    batch, sq, q_off, hq, hkv, dqk, dv, causal = case
    sk = q_off + sq if causal else 384
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(batch * sq, hq, dqk, device="cuda", generator=g).bfloat16().requires_grad_()
    k = torch.randn(batch * sk, hkv, dqk, device="cuda", generator=g).bfloat16().requires_grad_()
    v = torch.randn(batch * sk, hkv, dv, device="cuda", generator=g).bfloat16().requires_grad_()
    o = A.flash_attention(q, k, v, batch, causal, None, q_off if causal else 0)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = A.attention_ref(qr, kr, vr, batch, causal, None, q_off if causal else 0)
    o_ref.backward(do.float())
    assert (o.float() - o_ref.float()).abs().max().item() <= 2e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 3e-2 * b.abs().max().item() + 2e-2
        assert err <= tol, f"{name}: err {err} tol {tol}"


WINDOW_CASES = [
    # batch, seq, hq, hkv, d, window, sinks
    (1, 512, 4, 2, 128, 128, False),
    (1, 640, 2, 2, 128, 200, True),
    (2, 384, 4, 1, 64, 128, True),
    (1, 1024, 2, 1, 128, 300, False),
    (1, 256, 2, 2, 128, 1000, True),     # window longer than the sequence
    (1, 384, 4, 4, 128, 0, True),        # sinks only
]


@pytest.mark.parametrize("case", WINDOW_CASES)
def test_flash_attn_sliding_window_and_sinks(case):
    batch, seq, hq, hkv, d, window, with_sinks = case
    q, k, v = _inputs(batch, seq, hq, hkv, d, d, seed=5)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    sinks = (torch.randn(hq, device="cuda") * 2).requires_grad_() if with_sinks else None
    o = A.flash_attention(q, k, v, batch, True, None, 0, window, sinks)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sr = sinks.detach().clone().requires_grad_() if with_sinks else None
    o_ref, _ = A.attention_ref(qr, kr, vr, batch, True, None, 0, window, sr)
    o_ref.backward(do.float())
    assert (o.float() - o_ref.float()).abs().max().item() <= 2e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 3e-2 * b.abs().max().item() + 2e-2
        assert err <= tol, f"{name}: err {err} tol {tol}"
    if with_sinks:
        err = (sinks.grad - sr.grad).abs().max().item()
        assert err <= 3e-2 * sr.grad.abs().max().item() + 2e-2, (sinks.grad, sr.grad)


def test_packed_document_attention_forward_backward():
    """rope_attention with document segments (packed sequences) vs the fp32 reference run per document."""
    from primus_b200.ops import layers as L

    hq, hkv, d = 4, 2, 128
    T = 1024
    segs = [(0, 256), (256, 384), (384, 896), (896, 1024)]
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device="cuda", generator=g).bfloat16().requires_grad_()
    out = L.rope_attention(qkv, None, None, None, 1, hq, hkv, d, segments=segs)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    ref_in = qkv.detach().float().cpu().requires_grad_()
    ref = L.rope_attention(ref_in, None, None, None, 1, hq, hkv, d, segments=segs)
    ref.backward(do.float().cpu())
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    err = (qkv.grad.float().cpu() - ref_in.grad).abs().max().item()
    assert err <= 3e-2 * ref_in.grad.abs().max().item() + 2e-2, err


@pytest.mark.parametrize("case", [(1, 384, 4, 2, 128, 0, 30.0), (1, 512, 2, 2, 128, 200, 20.0), (2, 256, 4, 1, 64, 0, 50.0)])
def test_flash_attn_softcapped_scores(case):
    batch, seq, hq, hkv, d, window, cap = case
    q, k, v = _inputs(batch, seq, hq, hkv, d, d, seed=11)
    q, k = (q * 3).detach(), (k * 3).detach()                 # large scores, so that the cap bites
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = A.flash_attention(q, k, v, batch, True, None, 0, window, None, cap)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = A.attention_ref(qr, kr, vr, batch, True, None, 0, window, None, cap)
    o_ref.backward(do.float())
    assert (o.float() - o_ref.float()).abs().max().item() <= 3e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        tol = 4e-2 * b.abs().max().item() + 3e-2
        assert err <= tol, f"{name}: err {err} tol {tol}"
