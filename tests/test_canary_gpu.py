"""Out-of-bounds write check without a sanitizer: every output of a kernel is a slice in the middle of a larger buffer
filled with a sentinel, and the bytes before and after the slice must be untouched after the launch."""
import pytest
import torch

from primus_b200.ops import _lib, fp8, fused, gemm

pytestmark = pytest.mark.gpu

PAD = 4096  # bytes on each side (a multiple of every alignment the kernels ask for)


class Guarded:
    def __init__(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        self.nbytes = n * torch.empty(0, dtype=dtype).element_size()
        self.raw = torch.full((self.nbytes + 2 * PAD,), 0xA5, dtype=torch.uint8, device="cuda")
        self.t = self.raw[PAD:PAD + self.nbytes].view(dtype).view(*shape)

    def check(self, what):
        assert bool((self.raw[:PAD] == 0xA5).all()) and bool((self.raw[PAD + self.nbytes:] == 0xA5).all()), \
            f"{what}: bytes outside the output were written"
        assert not bool((self.raw[PAD:PAD + self.nbytes] == 0xA5).all()), f"{what}: output untouched"


def test_outputs_stay_inside_their_buffers():
    torch.manual_seed(0)
    # bf16 GEMM with edge tiles in M and N
    M, N, K = 384 + 64, 640 + 8, 256
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    out = Guarded((M, N), torch.bfloat16)
    gemm.gemm(a, b, out=out.t)
    torch.cuda.synchronize()
    out.check("gemm_bf16")
    assert torch.allclose(out.t.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    # RMSNorm forward: rows not a multiple of the rows-per-CTA
    rows, H = 1001, 4096
    x = torch.randn(rows, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    y, rstd = Guarded((rows, H), torch.bfloat16), Guarded((rows,), torch.float32)
    _lib.call("rmsnorm_fwd", x, None, w, y.t, None, rstd.t, rows, H, H, H, 1e-5)
    torch.cuda.synchronize()
    y.check("rmsnorm_fwd y")
    rstd.check("rmsnorm_fwd rstd")
    # SwiGLU forward
    T, I = 1001, 1408
    h1 = torch.randn(T, 2 * I, device="cuda").bfloat16()
    act = Guarded((T, I), torch.bfloat16)
    _lib.call("swiglu_fwd", h1, None, act.t, T, I, 0.0, 0)
    torch.cuda.synchronize()
    act.check("swiglu_fwd")
    # MXFP8 quantisation, both directions, and the tensor-wise variant
    R, C = 256, 384
    xq = torch.randn(R, C, device="cuda").bfloat16()
    for name in ("quant_mxfp8", "quant_fp8_tensorwise"):
        outs = [Guarded((R, C), torch.uint8), Guarded((R * C // 32,), torch.uint8),
                Guarded((R, C), torch.uint8), Guarded((R * C // 32,), torch.uint8)]
        if name == "quant_mxfp8":
            _lib.call(name, xq, R, C, *[o.t for o in outs])
        else:
            amax = Guarded((1,), torch.float32)
            _lib.call(name, xq, R, C, amax.t, *[o.t for o in outs])
        torch.cuda.synchronize()
        for i, o in enumerate(outs):
            o.check(f"{name} output {i}")
        ref = fp8.quantize_mxfp8_ref(xq, True, True, tensorwise=(name != "quant_mxfp8"))
        assert torch.equal(outs[0].t, ref.q_row) and torch.equal(outs[3].t, ref.sf_col)
    # RoPE in place on a guarded [T, heads, d] tensor
    Tr, h, d = 333, 4, 128
    q = Guarded((Tr, h, d), torch.bfloat16)
    q.t.copy_(torch.randn(Tr, h, d, device="cuda").bfloat16())
    cos, sin = fused.rope_tables(Tr, d, 10000.0, torch.device("cuda"))
    fused.rope_inplace_(q.t, cos, sin)
    torch.cuda.synchronize()
    q.check("rope")
    _lib.check_status()
