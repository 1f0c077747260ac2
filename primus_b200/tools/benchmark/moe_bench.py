"""MoE layer benchmark: forward + backward of one expert-parallel MoE layer, un-fused (NCCL all-to-all +
grouped GEMM) against the fused dispatch / combine kernels over symmetric memory.

    torchrun --nproc-per-node N -m primus_b200.tools.benchmark.moe_bench --model deepseek_v2_lite

Token shapes follow the reference's all-to-all benchmark table (hidden, sequence, top-k per model:
benchmark/kernel/rccl/benchmark_all2all.py:16-37).  Times are CUDA-event medians, max over ranks.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .common import emit, time_cuda

MODELS = {  # hidden, moe ffn, experts, top-k, tokens per rank
    "deepseek_v2_lite": (2048, 1408, 64, 6, 4096),
    "deepseek_v2": (5120, 1536, 160, 6, 4096),
    "deepseek_v3": (7168, 2048, 256, 8, 4096),
    "mixtral_8x7B": (4096, 14336, 8, 2, 4096),
    "qwen3_235B": (4096, 1536, 128, 8, 4096),
    "qwen3_30B_A3B": (2048, 768, 128, 8, 4096),
}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="deepseek_v2_lite", choices=sorted(MODELS))
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (to fit small EP sizes)")
    ap.add_argument("--capacity-factor", type=float, default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)

    from ...models.config import TransformerConfig
    from ...models.moe import MoELayer
    from ...ops import _lib
    from ...parallel import state as ps

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ps.initialize_model_parallel(ep=world)
    H, I, E, k, T = MODELS[args.model]
    T = args.tokens or T
    E = args.experts or E
    rows = []
    for fused in (False, True):
        cfg = TransformerConfig(num_layers=1, hidden_size=H, ffn_hidden_size=4 * H, num_attention_heads=H // 128,
                                vocab_size=1024, params_dtype="bf16", num_experts=E, moe_router_topk=k,
                                moe_ffn_hidden_size=I, moe_layer_freq=[1], moe_aux_loss_coeff=0.0, seq_length=T,
                                expert_model_parallel_size=world, use_turbo_mega_moe=fused,
                                moe_fused_capacity_factor=args.capacity_factor)
        torch.manual_seed(7)
        layer = MoELayer(cfg, 0, torch.device("cuda"), 1)
        for p in layer.parameters():
            p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        xs = [torch.randn(T, H, device="cuda").bfloat16().requires_grad_() for _ in range(4)]
        dys = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(4)]

        def step(i):
            x = xs[i % 4]
            x.grad = None
            layer(x).backward(dys[i % 4])

        def fwd(i):
            with torch.no_grad():
                layer(xs[i % 4])

        t_fb = time_cuda(step, args.iters, args.warmup)
        t_f = time_cuda(fwd, args.iters, args.warmup)
        torch.cuda.synchronize()
        _lib.check_status()
        vals = torch.tensor([t_fb["ms_median"], t_f["ms_median"]], device="cuda")
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        flops = 2.0 * T * k * 3 * H * I * 3   # fc1 (2I) + fc2 (I), forward + 2x backward
        rows.append({"model": args.model, "ep": world, "tokens/rank": T, "experts": E, "topk": k,
                     "path": "fused" if fused else ("nccl a2a" if world > 1 else "local"),
                     "fwd_ms": vals[1].item(), "fwd+bwd_ms": vals[0].item(),
                     "expert TFLOP/s/GPU": flops / (vals[0].item() * 1e-3) / 1e12})
    if not dist.is_initialized() or dist.get_rank() == 0:
        emit(rows, args.output, "MoE layer forward+backward")
    return rows


if __name__ == "__main__":
    main()
