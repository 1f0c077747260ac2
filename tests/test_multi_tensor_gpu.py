"""Multi-tensor apply kernels vs plain PyTorch."""
import pytest
import torch

from primus_b200.ops import multi_tensor as mt

pytestmark = pytest.mark.gpu


def _tensors(dtype, sizes=(1, 7, 65536, 65537, 200001, 33)):
    torch.manual_seed(0)
    return [torch.randn(n, device="cuda").to(dtype) for n in sizes]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_l2norm(dtype):
    ts = _tensors(dtype)
    tot, per = mt.multi_tensor_l2norm(ts, per_tensor=True)
    ref_per = torch.stack([t.float().norm() for t in ts])
    assert torch.allclose(per, ref_per, rtol=1e-4)
    assert torch.allclose(tot, ref_per.pow(2).sum().sqrt(), rtol=1e-4)
    tot2 = mt.multi_tensor_l2norm(ts)
    assert torch.equal(tot, tot2)  # deterministic reduction order


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float32, torch.float32)])
def test_scale_and_overflow_flag(src, dst):
    xs = _tensors(src)
    outs = [torch.empty_like(x, dtype=dst) for x in xs]
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    mt.multi_tensor_scale(xs, outs, 0.5, flag)
    for x, o in zip(xs, outs):
        assert torch.allclose(o.float(), (x.float() * 0.5).to(dst).float(), rtol=1e-6, atol=0)
    assert flag.item() == 0
    xs[3][5] = float("inf")
    mt.multi_tensor_scale(xs, outs, 0.5, flag)
    assert flag.item() == 1


def test_axpby():
    xs, ys = _tensors(torch.float32), [t * 3 for t in _tensors(torch.float32)]
    outs = [torch.empty_like(x, dtype=torch.bfloat16) for x in xs]
    mt.multi_tensor_axpby(xs, ys, outs, 2.0, -1.0)
    for x, y, o in zip(xs, ys, outs):
        assert torch.allclose(o.float(), (2.0 * x - y).bfloat16().float(), rtol=1e-6, atol=0)
