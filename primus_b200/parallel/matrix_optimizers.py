"""SGD (momentum) and Muon on top of the flat parameter / gradient buffers.

Both reuse :class:`DistributedOptimizer`'s machinery (fp32 master copy, global-norm clipping with the device-side
coefficient and skip flag, bf16 parameter write-back) and replace only the update rule.  They work on whole
parameters, so they require ``use_distributed_optimizer = False`` (every rank holds the full buffers).

Muon (momentum + Newton-Schulz orthogonalisation of the update of every 2-D hidden matrix; embeddings, the LM
head, 1-D parameters and expert stacks fall back to AdamW) follows the recipe the reference exposes through
its ``optimizer: muon`` keys (primus/configs/modules/megatron/trainer_base.yaml:101-111,
primus/backends/megatron/core/optimizer/per_head_muon.py): quintic iteration with coefficients
(3.4445, -4.7750, 2.0315), 5 steps, Nesterov momentum 0.95, update scaled by ``0.2 * sqrt(max(rows, cols))``
so that its RMS matches AdamW's and the same learning rate / weight decay can be used.  The matrix products run
on the tcgen05 GEMM (``ops/gemm.py``) for CUDA tensors.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from ..ops import optim as optim_ops
from .distributed import DistributedOptimizer

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(m: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate ``U V^T`` of ``m = U S V^T`` (fp32 in, fp32 out)."""
    a, b, c = NS_COEFFS
    transposed = m.shape[0] > m.shape[1]
    x = m.t() if transposed else m
    x = x / (x.norm() + 1e-7)
    use_kernel = x.is_cuda and x.shape[0] % 8 == 0 and x.shape[1] % 8 == 0
    x = x.contiguous().bfloat16() if use_kernel else x.contiguous()
    for _ in range(steps):
        if use_kernel:
            A = G.gemm(x, x, fp8=False)                                   # X X^T
            B = (b * A.float() + c * G.gemm(A, A, fp8=False).float()).bfloat16()
            x = (a * x.float() + G.gemm(B, x, b_mn=True, fp8=False).float()).bfloat16()
        else:
            A = x @ x.t()
            B = b * A + c * (A @ A)
            x = a * x + B @ x
    x = x.float()
    return x.t() if transposed else x


class _PerParameterOptimizer(DistributedOptimizer):
    def __init__(self, buffers, **kw):
        assert all(not b.use_distributed_optimizer for b in buffers), \
            "SGD / Muon update whole parameters: set use_distributed_optimizer to false"
        super().__init__(buffers, **kw)

    def _param_views(self):
        """(parameter, master view, gradient view, state dict of the bucket, offset in the bucket's state)."""
        for st in self.state:
            buf = st["buf"]
            for p in st["bucket"].params:
                o = buf.param_offsets[p]
                lo = o - st["s"]
                n = p.numel()
                yield p, st["master"][lo:lo + n].view(p.shape), buf.grad_data[o:o + n].view(p.shape), st, lo

    def _write_back(self):
        for st in self.state:
            st["buf"].param_data[st["s"]:st["e"]].copy_(st["master"])

    def step(self, lr=None, weight_decay=None, group_lr=None):
        assert not group_lr, "decoupled_lr / head_lr_mult are built for the Adam optimizer"
        lr = self.lr if lr is None else lr
        wd = self.weight_decay if weight_decay is None else weight_decay
        self.step_count += 1
        G.bump_weight_generation()
        self.compute_grad_norm()
        skip = bool(self.skip.item()) if self.check_for_nan else False   # one scalar read per step
        if not skip:
            self._update(lr, wd)
            self._write_back()
        if self.deosc is not None:
            self.deosc.run(self)
        return self.grad_norm


class SGD(_PerParameterOptimizer):
    def __init__(self, buffers, momentum: float = 0.9, **kw):
        super().__init__(buffers, **kw)
        self.momentum = momentum

    def _update(self, lr, wd):
        for p, master, grad, st, lo in self._param_views():
            g = grad * self.coef
            if wd and p.dim() > 1:
                g = g + wd * master
            mom = st["m"][lo:lo + p.numel()].view(p.shape)
            mom.mul_(self.momentum).add_(g)
            master.add_(mom, alpha=-lr)


class Muon(_PerParameterOptimizer):
    def __init__(self, buffers, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5, **kw):
        super().__init__(buffers, **kw)
        self.momentum, self.nesterov, self.ns_steps = momentum, nesterov, ns_steps

    @staticmethod
    def is_matrix(p) -> bool:
        return p.dim() == 2 and not getattr(p, "_embedding_like", False)   # embeddings / LM head: element-wise update

    def _update(self, lr, wd):
        b1, b2 = self.betas
        for p, master, grad, st, lo in self._param_views():
            n = p.numel()
            m = st["m"][lo:lo + n].view(p.shape)
            if self.is_matrix(p):
                g = grad * self.coef
                m.mul_(self.momentum).add_(g)
                u = g.add(m, alpha=self.momentum) if self.nesterov else m
                o = newton_schulz(u, self.ns_steps) * (0.2 * max(p.shape) ** 0.5)
                master.mul_(1.0 - lr * wd).add_(o, alpha=-lr)
            else:
                flat_master = st["master"][lo:lo + n]
                gview = st["buf"].grad_data[st["buf"].param_offsets[p]:st["buf"].param_offsets[p] + n]
                optim_ops.adamw_step_(flat_master, st["m"][lo:lo + n], st["v"][lo:lo + n], gview, None, lr=lr, beta1=b1,
                                      beta2=b2, eps=self.eps, weight_decay=0.0 if p.dim() <= 1 else wd,
                                      step=self.step_count, grad_scale=self.coef, skip=None)


def build(name: str, buffers, **kw):
    name = (name or "adam").lower()
    if name in ("adam", "adamw"):
        return DistributedOptimizer(buffers, **kw)
    if name == "sgd":
        return SGD(buffers, momentum=kw.pop("sgd_momentum", 0.9), **kw)
    if name == "muon":
        return Muon(buffers, momentum=kw.pop("muon_momentum", 0.95), nesterov=kw.pop("muon_use_nesterov", True),
                    ns_steps=kw.pop("muon_num_ns_steps", 5), **kw)
    raise ValueError(f"unknown optimizer {name!r}")
