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


def bench_kernels(args, H, I, E, k, T, world):
    """Device time of every stage of the fused path (forward), with the roofline of the two fused kernels:
    target = max(FLOPs / measured bf16 GEMM peak, bytes entering this GPU over NVLink / measured peer bandwidth)."""
    from ...ops import fused
    from ...ops import moe as moe_ops
    from ...parallel import fused_ep
    from ...parallel import state as ps
    from .fused_comm_bench import _max_over_ranks, _peaks

    st = ps.get_state()
    ws = fused_ep.get_workspace(st.ep_group if world > 1 else None, T, k, E, H, args.capacity_factor)
    torch.manual_seed(3 + (dist.get_rank() if dist.is_initialized() else 0))
    e_local = E // world
    x = torch.randn(T, H, device="cuda").bfloat16()
    logits = torch.randn(T, E, device="cuda")
    probs, idx, _ = moe_ops.router_scores(logits, k)
    w1 = (torch.randn(e_local, 2 * I, H, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(e_local, H, I, device="cuda") * 0.02).bfloat16()
    state = {}

    def f_plan(i):
        state["plan"] = ws.plan(idx, probs)

    def f_dispatch(i):
        state["plan"] = ws.plan(idx, probs)          # a dispatch always follows a plan (barrier protocol)
        state["xp"], state["h1"] = ws.dispatch_gemm(x, w1, state["plan"], False)

    def f_full(i):
        plan = ws.plan(idx, probs)
        xp, h1 = ws.dispatch_gemm(x, w1, plan, False)
        act = fused.swiglu(h1, plan.finalize().probs_perm, 0.0)
        state["out"] = ws.gemm_combine(act, w2, plan, False)

    t_plan = _max_over_ranks(time_cuda(f_plan, args.iters, args.warmup)["ms_median"])
    t_disp = _max_over_ranks(time_cuda(f_dispatch, args.iters, args.warmup)["ms_median"])
    t_full = _max_over_ranks(time_cuda(f_full, args.iters, args.warmup)["ms_median"])
    h1 = state["h1"]
    pp = state["plan"].finalize().probs_perm
    t_act = _max_over_ranks(time_cuda(lambda i: fused.swiglu(h1, pp, 0.0), args.iters, args.warmup)["ms_median"])
    torch.cuda.synchronize()
    _lib_check()
    peak, link = _peaks()
    rows_rank = T * k                      # balanced routing: every rank receives as many rows as it sends
    remote = rows_rank * (world - 1) / world * H * 2.0
    t_gemm1 = t_disp - t_plan
    t_gemm2 = t_full - t_disp - t_act
    out = []
    for name, t, fl in (("dispatch + GEMM1", t_gemm1, 2.0 * rows_rank * 2 * I * H),
                        ("GEMM2 + combine (+ local top-k sum)", t_gemm2, 2.0 * rows_rank * H * I)):
        target = max(fl / peak, remote / link) * 1e3
        out.append({"model": args.model, "ep": world, "stage": name, "ms": t, "roofline_ms": target,
                    "fraction_of_roofline": target / t, "bound": "compute" if fl / peak > remote / link else "nvlink"})
    out.append({"model": args.model, "ep": world, "stage": "routing plan (2 kernels + barrier)", "ms": t_plan})
    out.append({"model": args.model, "ep": world, "stage": "SwiGLU x prob", "ms": t_act})
    out.append({"model": args.model, "ep": world, "stage": "whole fused forward (no router)", "ms": t_full})
    return out


def _lib_check():
    from ...ops import _lib

    _lib.check_status()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--kernels", action="store_true", help="time the stages of the fused forward separately")
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
    if args.kernels:
        rows = bench_kernels(args, H, I, E, k, T, world)
        if not dist.is_initialized() or dist.get_rank() == 0:
            emit(rows, args.output, "fused expert-parallel forward, per stage")
        return rows
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
