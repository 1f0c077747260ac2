"""Memory-bound kernels (RMSNorm, RoPE, SwiGLU, cross-entropy, AdamW, norms) vs PyTorch fp32 references."""
import pytest
import torch

from primus_b200.ops import fused as F
from primus_b200.ops import optim as O

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= atol + rtol * b.abs().max().item(), f"err {err}"


@pytest.mark.parametrize("H", [128, 256, 4096, 2048 + 64, 7168, 8192, 16384])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(H, with_res):
    T = 300
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(T, H, device="cuda").bfloat16().requires_grad_() if with_res else None
    w = torch.nn.Parameter((1 + 0.1 * torch.randn(H, device="cuda")).bfloat16())
    out = F.rmsnorm(x, w, 1e-5, r)
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    xs = xr + rr if with_res else xr
    yr = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    if with_res:
        y, xsum = out
        dy, ds = torch.randn_like(y), torch.randn_like(xsum)
        torch.autograd.backward([y, xsum], [dy, ds])
        torch.autograd.backward([yr, xs], [dy.float(), ds.float()])
        _close(xsum, xs)
        _close(r.grad, rr.grad)
    else:
        y = out
        dy = torch.randn_like(y)
        y.backward(dy)
        yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, rtol=2e-2, atol=0.3)


def test_rmsnorm_main_grad_accumulates():
    T, H = 1000, 1024
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = torch.nn.Parameter(torch.ones(H, device="cuda").bfloat16())
    w.main_grad = torch.zeros(H, device="cuda")
    for _ in range(2):
        F.rmsnorm(x, w, 1e-5).backward(torch.ones(T, H, device="cuda").bfloat16())
    xr = x.detach().float()
    ref = 2 * (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5)).sum(0)
    _close(w.main_grad, ref, rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("rot", [128, 64])
def test_rope(rot):
    T, h, d = 257, 6, 128
    cos, sin = F.rope_tables(512, rot, 10000.0, "cuda")
    x = torch.randn(T, h, d, device="cuda").bfloat16().requires_grad_()
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    y = F.rope(x, cos, sin, pos, rot)
    ref = F.rope_ref(x.detach(), cos, sin, pos, rot)
    _close(y, ref)
    dy = torch.randn_like(y)
    y.backward(dy)
    gref = F.rope_ref(dy, cos, -sin, pos, rot)
    _close(x.grad, gref)


@pytest.mark.parametrize("probs,clamp", [(False, 0.0), (True, 0.0), (True, 7.0)])
def test_swiglu(probs, clamp):
    T, I = 333, 1408
    x = (3 * torch.randn(T, 2 * I, device="cuda")).bfloat16().requires_grad_()
    p = torch.rand(T, device="cuda").requires_grad_() if probs else None
    y = F.swiglu(x, p, clamp)
    xr = x.detach().float().requires_grad_()
    pr = p.detach().clone().requires_grad_() if probs else None
    g, u = xr[:, :I], xr[:, I:]
    if clamp > 0:
        g, u = g.clamp(max=clamp), u.clamp(-clamp, clamp)
    yr = torch.nn.functional.silu(g) * u
    if probs:
        yr = yr * pr[:, None]
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    if probs:
        _close(p.grad, pr.grad, rtol=2e-2, atol=0.5)


@pytest.mark.parametrize("V", [32000, 128256])
def test_cross_entropy(V):
    T = 64
    logits = (2 * torch.randn(T, V, device="cuda")).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    lr = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, labels, reduction="none")
    scale = torch.rand(T, device="cuda")
    (ref * scale).sum().backward()
    lg = logits.clone().requires_grad_()
    loss = F.cross_entropy(lg, labels)
    (loss * scale).sum().backward()
    _close(loss, ref, rtol=1e-3, atol=1e-2)
    assert (lg.grad.float() - lr.grad).abs().max().item() <= 1e-2


def test_adamw_and_norms():
    n = 1_000_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ss = torch.zeros(1, device="cuda")
    coef = torch.zeros(1, device="cuda")
    nrm = torch.zeros(1, device="cuda")
    for step in (1, 2, 3):
        O.sumsq_(g, ss)
        O.clip_coef_(ss, 1.0, coef, nrm)
        ref.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref], 1.0)
        opt.step()
        O.adamw_step_(p, m, v, g, pb, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                      grad_scale=coef)
    assert abs(nrm.item() - g.norm().item()) <= 1e-3 * g.norm().item()
    _close(p, ref.detach(), rtol=1e-4, atol=1e-5)
    _close(pb, ref.detach(), rtol=1e-2, atol=1e-2)
    # skip flag leaves state untouched
    before = p.clone()
    skip = torch.ones(1, device="cuda", dtype=torch.int32)
    O.adamw_step_(p, m, v, g, pb, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=4, skip=skip)
    assert torch.equal(p, before)
    # bf16 gradients
    gb = g.bfloat16()
    O.sumsq_(gb, ss)
    assert abs(ss.item() - gb.float().pow(2).sum().item()) <= 1e-3 * ss.item()


def test_embedding_backward_main_grad():
    V, H, T = 1000, 256, 4096
    w = torch.nn.Parameter(torch.randn(V, H, device="cuda").bfloat16())
    w.main_grad = torch.zeros(V, H, device="cuda")
    tok = torch.randint(0, V, (T,), device="cuda")
    y = F.embedding(tok, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, tok, dy.float())
    _close(w.main_grad, ref, rtol=1e-3, atol=1e-3)


def test_chunked_linear_cross_entropy_matches_full_gpu():
    """Chunked linear + cross entropy (no [tokens, vocab] logits) gives the loss trajectory of the plain path."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import _lib
    from primus_b200.parallel import state as ps

    res = {}
    for chunk in (0, 128):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2, vocab_size=2048,
                               params_dtype="bf16", seq_length=256, cross_entropy_chunk_tokens=chunk)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=256, train_iters=4, lr=1e-3,
                         lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1)
        torch.manual_seed(0)
        tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
        res[chunk] = tr.train()
        torch.cuda.synchronize()
        _lib.check_status()
    assert all(abs(a - b) <= 5e-3 * max(1.0, abs(a)) for a, b in zip(res[0], res[128])), res


def test_softcap_forward_backward():
    from primus_b200.ops import fused

    torch.manual_seed(0)
    x = (torch.randn(512, 1024, device="cuda") * 20).bfloat16().requires_grad_()
    y = fused.softcap(x, 30.0)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = torch.tanh(xr / 30.0) * 30.0
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("with_probs", [False, True])
def test_gated_unit_activations(act, with_probs):
    """SwiGLU / GEGLU (optionally weighted by routing probabilities) forward and backward vs the fp32 reference."""
    from primus_b200.ops import fused

    torch.manual_seed(1)
    T, I = 384, 256
    x = torch.randn(T, 2 * I, device="cuda").bfloat16().requires_grad_()
    p = torch.rand(T, device="cuda").requires_grad_() if with_probs else None
    y = fused.swiglu(x, p, 0.0, act)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    pr = p.detach().clone().requires_grad_() if with_probs else None
    yr = fused.swiglu_ref(xr, pr, 0.0, act)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    if with_probs:
        torch.testing.assert_close(p.grad, pr.grad, rtol=3e-2, atol=0.3)


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_adamw_kernel_state_dtypes(state_dtype, grad_dtype):
    """AdamW kernel with fp32 / bf16 moments and gradients vs the plain PyTorch path on the same values."""
    from primus_b200.ops import optim

    torch.manual_seed(2)
    n = 4096 * 3 + 5
    master = torch.randn(n, device="cuda")
    m = (torch.randn(n, device="cuda") * 0.01).to(state_dtype)
    v = (torch.rand(n, device="cuda") * 1e-4).to(state_dtype)
    g = torch.randn(n, device="cuda").to(grad_dtype)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    ref = [t.detach().cpu().clone() for t in (master, m, v, g)]
    ref_out = torch.empty(n, dtype=torch.bfloat16)
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
    optim.adamw_step_(master, m, v, g, out, **kw)
    optim.adamw_step_(ref[0], ref[1], ref[2], ref[3], ref_out, **kw)
    torch.cuda.synchronize()
    tol = 1e-5 if state_dtype == torch.float32 else 1e-2
    torch.testing.assert_close(master.cpu(), ref[0], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(m.cpu().float(), ref[1].float(), rtol=tol, atol=1e-6)
    torch.testing.assert_close(v.cpu().float(), ref[2].float(), rtol=tol, atol=1e-9)
    torch.testing.assert_close(out.cpu().float(), ref_out.float(), rtol=1e-2, atol=1e-2)
