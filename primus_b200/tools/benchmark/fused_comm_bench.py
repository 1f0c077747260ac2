"""Fused compute+collective kernels against their NCCL compositions, with roofline fractions.

    torchrun --nproc-per-node N -m primus_b200.tools.benchmark.fused_comm_bench [--suite tp|tp-fp8|dp|all] [--model llama3.1_70B]

* ``tp``: all-gather -> GEMM and GEMM -> reduce-scatter (``csrc/gemm_tp_fused.cu``) at the tensor-parallel shapes
  of the model (QKV / FC1 column-parallel, proj / FC2 row-parallel, sequence parallel) vs ``NCCL collective + GEMM``;
* ``dp``: reduce-scatter + AdamW + all-gather over peer memory (``csrc/dp_fused.cu``) vs NCCL reduce-scatter +
  AdamW kernel + NCCL all-gather on a flat buffer of ``--dp-params`` parameters.

Every time is a CUDA-event median, maximum over ranks.  Roofline: target = max(FLOPs / measured bf16 GEMM peak,
bytes that must cross NVLink per GPU / measured per-direction peer bandwidth); fraction = target / achieved.
Peaks come from ``MEASURED_PEAKS.json`` next to the repository root when present (else 1590 TFLOP/s, 770 GB/s).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from .common import emit, time_cuda


def _peaks():
    p = Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"
    tf, link = 1590.0, 770.0
    if p.exists():
        try:
            d = json.loads(p.read_text())
            tf = float(d.get("bf16_tflops", tf))
            link = float(d.get("nvlink_peer_gbs", link))
        except Exception:  # noqa: BLE001
            pass
    return tf * 1e12, link * 1e9


def _max_over_ranks(v: float) -> float:
    t = torch.tensor([v], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_tp(model: str, tokens: int, iters: int):
    from ...core.config.presets import load_preset
    from ...models.config import TransformerConfig
    from ...parallel import fused_tp

    world = dist.get_world_size()
    cfg = TransformerConfig.from_dict(load_preset(model, "models"))
    h, ffn = cfg.hidden_size, cfg.ffn_hidden_size
    group = dist.group.WORLD
    peak, link = _peaks()
    shapes = [("qkv  (AG->GEMM)", "ag", cfg.qkv_width // world, h), ("fc1  (AG->GEMM)", "ag", 2 * ffn // world, h),
              ("proj (GEMM->RS)", "rs", h, cfg.num_attention_heads * cfg.kv_channels // world),
              ("fc2  (GEMM->RS)", "rs", h, ffn // world)]
    rows = []
    for name, kind, N, K in shapes:
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        if kind == "ag":
            xs = [torch.randn(tokens // world, K, device="cuda").bfloat16() for _ in range(4)]
            fn = lambda fused: (lambda i: fused_tp.ag_gemm(xs[i % 4], w, group, fused=fused))
        else:
            xs = [torch.randn(tokens, K, device="cuda").bfloat16() for _ in range(4)]
            fn = lambda fused: (lambda i: fused_tp.gemm_rs(xs[i % 4], w, group, fused=fused))
        t_f = _max_over_ranks(time_cuda(fn(True), iters)["ms_median"])
        t_n = _max_over_ranks(time_cuda(fn(False), iters)["ms_median"])
        ctx = fused_tp.get_context(group)
        inst = ctx.instance(0 if kind == "ag" else 1, tokens, N, K)
        flops = 2.0 * tokens * N * K
        # bytes entering (AG) / leaving towards the owners (RS) each GPU over NVLink
        nv = (tokens // world) * (world - 1) * (K if kind == "ag" else N) * 2.0
        target = max(flops / peak, nv / link) * 1e3
        rows.append({"op": name, "tp": world, "M": tokens, "N/rank" if kind == "ag" else "N": N, "K": K,
                     "copy_ctas": fused_tp._comm_ctas(ctx, inst), "fused_ms": t_f, "nccl+gemm_ms": t_n, "speedup": t_n / t_f,
                     "roofline_ms": target,
                     "fraction_of_roofline": target / t_f, "bound": "compute" if flops / peak > nv / link else "nvlink"})
    return rows


def bench_tp_fp8(model: str, tokens: int, iters: int, emulate_tp: int = 0):
    """MXFP8 recipe under sequence parallelism: all-gather of the quantised shard + MXFP8 GEMM against all-gather of
    the bf16 shard + quantisation of the gathered tensor + the same GEMM.  ``emulate_tp`` > world: the weight shard has
    the width of that tensor-parallel size (the gathered tensor still has ``tokens`` rows)."""
    from ...core.config.presets import load_preset
    from ...models.config import TransformerConfig
    from ...ops import gemm as gemm_ops
    from ...parallel import fused_tp

    world = dist.get_world_size()
    tp = max(emulate_tp, world)
    cfg = TransformerConfig.from_dict(load_preset(model, "models"))
    h, ffn = cfg.hidden_size, cfg.ffn_hidden_size
    group = dist.group.WORLD
    rows = []
    gemm_ops.set_fp8_recipe("mxfp8")
    try:
        for name, N, K in (("qkv fprop", cfg.qkv_width // tp, h), ("fc1 fprop", 2 * ffn // tp, h)):
            N = N // 128 * 128
            w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
            w._is_weight = True
            xs = [torch.randn(tokens // world, K, device="cuda").bfloat16() for _ in range(4)]
            res = {}
            for mode in (True, False):
                fused_tp.QUANTIZED_GATHER = mode
                res[mode] = _max_over_ranks(time_cuda(lambda i: fused_tp.ag_gemm(xs[i % 4], w, group, fused=False), iters)["ms_median"])
            fused_tp.QUANTIZED_GATHER = True
            gather_bf16 = (tokens // world) * (world - 1) * K * 2.0
            rows.append({"op": name + " (MXFP8, AG + GEMM)", "ranks": world, "weight shard of tp": tp, "M": tokens, "N/rank": N,
                         "K": K, "quantised_gather_ms": res[True], "bf16_gather_ms": res[False],
                         "speedup": res[False] / res[True], "nvlink_MB_in_bf16": gather_bf16 / 1e6,
                         "nvlink_MB_in_mxfp8": gather_bf16 * (1 + 1 / 32) / 2 / 1e6})
    finally:
        gemm_ops.set_fp8_recipe(None)
    return rows


def bench_dp(n_params: int, iters: int):
    from ...ops import _lib
    from ...ops import optim as optim_ops
    from ...ops.fused import scratch
    from ...parallel.symm_mem import SymmetricBuffer

    world, rank = dist.get_world_size(), dist.get_rank()
    group = dist.group.WORLD
    n = n_params // (world * 1024) * (world * 1024)
    shard = n // world
    dev = torch.device("cuda", torch.cuda.current_device())
    sym_g = SymmetricBuffer(n * 4, group, dev)
    sym_p = SymmetricBuffer(n * 2, group, dev)
    grads = sym_g.local(torch.float32, n)
    params = sym_p.local(torch.bfloat16, n)
    grads.normal_()
    master = torch.randn(shard, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    red = torch.empty(shard, device=dev)
    sumsq = torch.zeros(1, device=dev)
    coef = torch.ones(1, device=dev)
    skip = torch.zeros(1, dtype=torch.int32, device=dev)
    P = _lib.call_ret("dp_num_partials")
    tg = (ctypes.c_long * world)(*[sym_g.peer_ptr(r) for r in range(world)])
    tp_ = (ctypes.c_long * world)(*[sym_p.peer_ptr(r) for r in range(world)])
    s0 = rank * shard

    def fused(i):
        sym_g.barrier(0)
        _lib.call("dp_reduce_scatter", tg, world, rank, s0, shard, red, 1.0 / world, scratch(dev, "dp_partials", P), sumsq, 0)
        sym_g.barrier(1)
        _lib.call("dp_adamw_allgather", tp_, world, rank, s0, shard, master, m, v, red, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1,
                  0.05, coef, skip)
        sym_p.barrier(0)

    g2 = torch.randn(n, device=dev)
    p2 = torch.empty(n, dtype=torch.bfloat16, device=dev)

    def nccl(i):
        dist.reduce_scatter_tensor(red, g2, group=group)
        optim_ops.sumsq_(red, sumsq, accumulate=False)
        optim_ops.adamw_step_(master, m, v, red, p2[s0:s0 + shard], lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                              weight_decay=0.1, step=10, grad_scale=coef, skip=skip)
        dist.all_gather_into_tensor(p2, p2[s0:s0 + shard], group=group)

    t_f = _max_over_ranks(time_cuda(fused, iters)["ms_median"])
    t_n = _max_over_ranks(time_cuda(nccl, iters)["ms_median"])
    torch.cuda.synchronize()
    _lib.check_status()
    _, link = _peaks()
    # per GPU over NVLink: read (world-1) remote shards of fp32 gradients, write the bf16 shard to (world-1) peers
    nv = shard * (world - 1) * (4.0 + 2.0)
    target = nv / link * 1e3
    return [{"op": "grad RS + AdamW + param AG", "dp": world, "params": n, "fused_ms": t_f, "nccl_ms": t_n,
             "speedup": t_n / t_f, "roofline_ms": target, "fraction_of_roofline": target / t_f, "bound": "nvlink"}]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--suite", default="all", choices=["tp", "tp-fp8", "dp", "all"])
    ap.add_argument("--emulate-tp", type=int, default=0, help="tp-fp8: width of the weight shard as under this TP size")
    ap.add_argument("--model", default="llama3.1_70B")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dp-params", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    if not dist.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rows = []
    if a.suite in ("tp", "all"):
        rows += bench_tp(a.model, a.tokens, a.iters)
    if a.suite == "tp-fp8":
        rows += bench_tp_fp8(a.model, a.tokens, a.iters, a.emulate_tp)
    if a.suite in ("dp", "all"):
        rows += bench_dp(a.dp_params, a.iters)
    if dist.get_rank() == 0:
        emit(rows, a.output, f"fused compute+collective kernels, {dist.get_world_size()} GPUs")
    dist.barrier()
    return rows


if __name__ == "__main__":
    main()
