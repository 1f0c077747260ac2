"""Flat-buffer optimizer kernels: fused AdamW (fp32 master/moments, bf16 param write-back, device-side
clip coefficient and skip flag so a step needs no host sync), sum of squares for the gradient norm,
and small cast / scale helpers.  CPU tensors run equivalent PyTorch code.

Parity: FusedAdam swap-in primus/backends/megatron/patches/torch_fused_adam_patches.py:40-88; gradient
clipping / found-inf handling of Megatron's distributed optimizer (primus/configs/modules/megatron/
trainer_base.yaml:72-118).
"""
from __future__ import annotations

import torch

from . import _lib
from .fused import scratch


def adamw_step_(master, exp_avg, exp_avg_sq, grad, param_out, *, lr, beta1, beta2, eps, weight_decay,
                step, grad_scale=None, skip=None):
    """In-place AdamW on flat state: fp32 master weights, fp32 or bf16 moments (both the same dtype).  ``grad`` fp32
    or bf16 (flat); ``param_out`` bf16 or None.

    ``grad_scale``: 1-element fp32 tensor multiplied into the gradient (clip coefficient);
    ``skip``: 1-element int32 tensor, non-zero -> the update is skipped (non-finite gradients)."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = master.numel()
    if not master.is_cuda:
        if skip is not None and int(skip.item()) != 0:
            return
        g = grad.float()
        if grad_scale is not None:
            g = g * grad_scale.float()
        m32 = exp_avg.float().mul_(beta1).add_(g, alpha=1 - beta1)
        v32 = exp_avg_sq.float().mul_(beta2).addcmul_(g, g, value=1 - beta2)
        exp_avg.copy_(m32)
        exp_avg_sq.copy_(v32)
        denom = (v32 / bc2).sqrt_().add_(eps)
        master.mul_(1 - lr * weight_decay).addcdiv_(m32 / bc1, denom, value=-lr)
        if param_out is not None:
            param_out.copy_(master.to(param_out.dtype))
        return
    assert master.dtype == torch.float32 and master.is_contiguous()
    assert grad.numel() == n and grad.is_contiguous()
    if param_out is not None:
        assert param_out.dtype == torch.bfloat16 and param_out.numel() == n
    assert exp_avg.dtype == exp_avg_sq.dtype and exp_avg.dtype in (torch.float32, torch.bfloat16)
    _lib.call("adamw_ex", master, exp_avg, exp_avg_sq, grad, int(grad.dtype == torch.bfloat16),
              int(exp_avg.dtype == torch.bfloat16), param_out, n,
              float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(bc1), float(bc2),
              grad_scale, skip)


def sumsq_(x, out, accumulate=False, nonfinite=None):
    """out[0] (+)= sum(x^2) in fp32 (deterministic two-stage reduction)."""
    if not x.is_cuda:
        s = x.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
        if nonfinite is not None and not torch.isfinite(out[0]):
            nonfinite.fill_(1)
        return out
    assert x.is_contiguous()
    P = _lib.call_ret("sumsq_num_partials")
    sc = scratch(x.device, "sumsq", P)
    _lib.call("sumsq", x, int(x.dtype == torch.bfloat16), x.numel(), sc, out, int(accumulate), nonfinite)
    return out


def clip_coef_(sumsq, max_norm, coef, norm_out=None, extra=1.0):
    """coef = min(1, max_norm/(sqrt(sumsq)+1e-6)) * extra, all on device."""
    if not sumsq.is_cuda:
        nrm = sumsq[0].sqrt()
        if norm_out is not None:
            norm_out[0] = nrm
        c = torch.clamp(max_norm / (nrm + 1e-6), max=1.0) if max_norm > 0 else torch.tensor(1.0)
        coef[0] = c * extra
        return coef
    _lib.call("clip_coef", sumsq, float(max_norm), float(extra), coef, norm_out)
    return coef


def cast_f32_to_bf16_(src, dst):
    if not src.is_cuda:
        dst.copy_(src.to(dst.dtype))
        return dst
    _lib.call("cast_f32_bf16", src, dst, src.numel())
    return dst
