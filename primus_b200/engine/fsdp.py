"""Fully sharded data parallelism (``use_torch_fsdp2``): parameters, gradients and optimizer state sharded over the
data-parallel ranks with PyTorch's ``fully_shard``; the layers still run this package's kernels on the gathered
parameters.

Every transformer layer is one sharding unit (parameters all-gathered right before the layer runs and freed after,
gradients reduce-scattered in fp32 after its backward), the root module holds the embedding, the final norm and the
output layer.  Sharded parameters and Adam state are fp32, compute parameters bf16.  Role of the reference's
``core/distributed/torch_fully_sharded_data_parallel.py`` and ``optimizer/fsdp2_fp32_master_weight_opt``; scope: data
parallelism only (tp = pp = cp = ep = 1), bf16 compute (no MXFP8 recipe), AdamW.  Checkpoints: the parameters are
written whole (gathered; ``engine/checkpoint.py``), each rank saves its own shards of the Adam moments.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_model(model: torch.nn.Module, device: torch.device, compute_dtype: torch.dtype, replicate_degree: int = 1):
    """``replicate_degree`` > 1: hybrid sharding (HSDP) -- the ranks form ``replicate_degree`` groups; parameters and
    optimizer state are sharded inside a group (consecutive ranks: the NVLink domain) and replicated across the groups,
    gradients are reduce-scattered inside and all-reduced across.  The reference's ``data_parallel_replicate_degree``
    (primus/backends/megatron/patches/args/hsdp_args_patches.py:12-70)."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    world = dist.get_world_size()
    if replicate_degree > 1:
        assert world % replicate_degree == 0, f"data_parallel_replicate_degree {replicate_degree} must divide {world} ranks"
        mesh = init_device_mesh(device.type, (replicate_degree, world // replicate_degree),
                                mesh_dim_names=("replicate", "shard"))
    else:
        mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp",))
    model.float()                                   # sharded (master) parameters are fp32
    # inputs are not cast: the layers receive fp32 rotary tables and integer position ids next to the bf16 activations
    mp = MixedPrecisionPolicy(param_dtype=compute_dtype if compute_dtype != torch.float32 else None,
                              reduce_dtype=torch.float32, cast_forward_inputs=False)
    for layer in model.decoder.layers.values():
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    return model


class FSDP2Optimizer:
    """AdamW over the sharded fp32 parameters with the interface the trainer uses (``step(lr, weight_decay)``,
    ``grad_norm``, ``compute_grad_norm``, ``zero_grad``).  1-D parameters (norm weights) get no weight decay."""

    def __init__(self, model, lr, betas, eps, weight_decay, clip_grad, check_for_nan=True):
        self.model = model
        self.clip_grad = clip_grad
        self.check_for_nan = check_for_nan
        decay = [p for p in model.parameters() if p.ndim > 1]
        no_decay = [p for p in model.parameters() if p.ndim <= 1]
        dev = next(model.parameters()).device
        self.opt = torch.optim.AdamW(
            [dict(params=decay, weight_decay=weight_decay), dict(params=no_decay, weight_decay=0.0)],
            lr=lr, betas=betas, eps=eps, fused=dev.type == "cuda")
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.state = []
        self.step_count = 0

    def zero_grad(self):
        self.opt.zero_grad(set_to_none=True)

    # ------------------------------------------------------------------ checkpoint: this rank's shards of the moments
    def state_dict(self):
        shards = []
        for name, p in self.model.named_parameters():
            st = self.opt.state.get(p)
            if not st:
                continue
            shards.append({"name": name, "step": float(st["step"]),
                           "exp_avg": _local(st["exp_avg"]).clone(), "exp_avg_sq": _local(st["exp_avg_sq"]).clone()})
        return {"step_count": self.step_count, "shards": shards}

    def load_state_dict(self, sd):
        by_name = dict(self.model.named_parameters())
        fused = bool(self.opt.param_groups[0].get("fused"))
        for s in sd["shards"]:
            p = by_name[s["name"]]
            self.opt.state[p] = {
                "step": torch.tensor(float(s["step"]), dtype=torch.float32, device=p.device if fused else "cpu"),
                "exp_avg": _like(p, s["exp_avg"]), "exp_avg_sq": _like(p, s["exp_avg_sq"])}
        self.step_count = int(sd.get("step_count", 0))

    def compute_grad_norm(self):
        n = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip_grad if self.clip_grad else float("inf"))
        n = n.full_tensor() if hasattr(n, "full_tensor") else n
        self.grad_norm.copy_(n.reshape(1).float())
        return self.grad_norm

    def step(self, lr=None, weight_decay=None):
        from ..ops import gemm

        norm = self.compute_grad_norm()
        if self.check_for_nan and not bool(torch.isfinite(norm).item()):
            self.zero_grad()
            return False
        for i, g in enumerate(self.opt.param_groups):
            if lr is not None:
                g["lr"] = lr
            if weight_decay is not None and i == 0:
                g["weight_decay"] = weight_decay
        self.opt.step()
        self.step_count += 1
        gemm.bump_weight_generation()
        return True


def _local(t):
    return t.to_local() if hasattr(t, "to_local") else t


def _like(p, local):
    """A moment tensor laid out like parameter ``p`` (sharded the same way) from this rank's saved shard."""
    local = local.to(device=p.device, dtype=torch.float32)
    if hasattr(p, "to_local"):
        from torch.distributed.tensor import DTensor

        return DTensor.from_local(local, p.device_mesh, p.placements, run_check=False, shape=p.shape, stride=p.stride())
    return local
