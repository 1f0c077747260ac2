"""tcgen05 bf16 GEMM vs a plain PyTorch fp32 reference: all operand layouts, output modes,
ragged shapes, and the autograd linear."""
import pytest
import torch

from primus_b200.ops import _lib
from primus_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


def _mk(M, N, K, a_mn, b_mn, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).bfloat16()
    return a, b


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 192), (384, 128, 1024), (1000, 776, 520), (8, 8, 8)])
@pytest.mark.parametrize("bn", [256, 128])
def test_gemm_layouts(a_mn, b_mn, shape, bn):
    M, N, K = shape
    a, b = _mk(M, N, K, a_mn, b_mn)
    G._BLOCK_N_OVERRIDE = bn
    try:
        d = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    finally:
        G._BLOCK_N_OVERRIDE = None
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (d.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-3
    assert err <= tol, f"max err {err} tol {tol}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
def test_gemm_fp32_out_and_accumulate(a_mn, b_mn):
    M, N, K = 512, 384, 2048
    a, b = _mk(M, N, K, a_mn, b_mn, seed=1)
    ref = _ref(a, b, a_mn, b_mn)
    d = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert (d - ref).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-3
    base = torch.randn(M, N, device="cuda")
    acc = base.clone()
    G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
    G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
    torch.cuda.synchronize()
    _lib.check_status()
    exp = base + 2 * ref
    assert (acc - exp).abs().max().item() <= 1e-3 * exp.abs().max().item() + 1e-3


def test_gemm_large_multiwave_and_deterministic():
    M, N, K = 4096, 6144, 4096
    a, b = _mk(M, N, K, False, False, seed=2)
    d1 = G.gemm(a, b)
    d2 = G.gemm(a, b)
    ref = (a.float() @ b.float().t())
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(d1, d2)
    assert (d1.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_linear_autograd_with_main_grad():
    T, I, O = 512, 1024, 768
    x = torch.randn(T, I, device="cuda").bfloat16().requires_grad_()
    w = torch.nn.Parameter((torch.randn(O, I, device="cuda") * 0.05).bfloat16())
    w.main_grad = torch.zeros(O, I, device="cuda")
    y = G.linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    assert (y.float() - yr).abs().max().item() <= 2e-2 * yr.abs().max().item()
    assert (x.grad.float() - xr.grad).abs().max().item() <= 2e-2 * xr.grad.abs().max().item()
    assert (w.main_grad - wr.grad).abs().max().item() <= 2e-3 * wr.grad.abs().max().item() + 1e-3
    assert w.grad is None
