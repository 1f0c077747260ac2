"""Headline benchmark: Llama-3.1-8B pre-training throughput (tokens/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 3 --warmup 3

Config (weak scaling): 32 layers, hidden 4096, 32/8 heads, FFN 14336, vocab 128256, seq 8192, micro-batch 1,
global batch 16 x N (128 at N=8), data parallel with the distributed optimizer, bf16 compute with fp32
master weights / main grads, synthetic uniform-random tokens, random-init N(0, 0.02) weights.

Two timed regions, both on the device with CUDA events, max over ranks:
  value : K optimizer steps back to back (inputs still arrive from pinned host memory on a side stream);
  e2e   : K further steps through ``Trainer.train`` which also reads every step's loss back to the host.
Rank 0 prints one JSON line.  ``--impl reference`` runs the reference's own CLI (TorchTitan backend) from
``baseline/_ref`` on the same model and batch, or says why it cannot.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOK_S_GPU = 16224.0  # Llama-3.1-8B, seq 8192, published by the reference for 8x MI325X (FP8)

MODELS = {
    "llama3.1_8B": dict(num_layers=32, hidden_size=4096, ffn_hidden_size=14336, num_attention_heads=32,
                        num_query_groups=8, kv_channels=128, vocab_size=128256, rotary_base=500000.0,
                        norm_epsilon=1e-5, max_position_embeddings=131072),
    "llama_tiny": dict(num_layers=4, hidden_size=1024, ffn_hidden_size=2816, num_attention_heads=8,
                       num_query_groups=4, kv_channels=128, vocab_size=32000),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._reader, daemon=True).start()
        except OSError:
            self.proc = None

    def _reader(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


def _reference_unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _reference_tokenizer_assets(path: Path) -> None:
    """Word-level tokenizer files for the reference's mock data: its mock corpus is text made of space-separated
    integers below 32000 (primus/backends/torchtitan/patches/mock_dataset_patches.py:28), and no Llama tokenizer can
    be downloaded here.  Every integer maps to its own id, so the token stream is uniform random."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    path.mkdir(parents=True, exist_ok=True)
    vocab = {str(i): i for i in range(32000)}
    vocab.update({"<unk>": 32000, "<s>": 32001, "</s>": 32002})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.add_special_tokens(["<s>", "</s>"])
    tok.save(str(path / "tokenizer.json"))
    (path / "tokenizer_config.json").write_text(json.dumps(
        {"bos_token": "<s>", "eos_token": "</s>", "add_bos_token": True, "add_eos_token": True}))


def reference_arm(args) -> int:
    """Runs the unmodified reference (copied to ``baseline/_ref``) through its own CLI and its TorchTitan backend
    (primus/cli/main.py -> primus/backends/torchtitan/torchtitan_pretrain_trainer.py:41): Llama-3.1-8B, seq 8192,
    micro-batch 1, the same global batch, bf16 FSDP2 + torch.compile, mock data.  Its Megatron backend (the one its
    published number comes from) cannot run: the Megatron-LM submodule directory is empty and Transformer-Engine /
    Primus-Turbo are not installed.  Throughput comes from the reference's own per-step log line (``tps`` = tokens
    per second per device, averaged since the previous line; it is logged every step, after the loss is read back)."""
    import importlib.util
    import re
    import tempfile

    root = Path(__file__).resolve().parent
    ref = root / "baseline" / "_ref"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.model != "llama3.1_8B":
        return _reference_unavailable("reference arm is wired for llama3.1_8B only")
    cfg = ref / "examples" / "torchtitan" / "configs" / "MI300X" / "llama3.1_8B-BF16-pretrain.yaml"
    if not cfg.exists():
        return _reference_unavailable(
            "reference (AMD-AGI/Primus) is not present under baseline/_ref: pip cannot build it offline (its build "
            "backend hatchling is not in the wheelhouse) and no copy of its package tree was placed there")
    spec = importlib.util.find_spec("torchtitan")
    if spec is None:
        return _reference_unavailable("reference TorchTitan backend needs the torchtitan package; its Megatron "
                                      "backend needs Megatron-LM, whose submodule directory is empty")
    backend_path = str(Path(spec.origin).parent.parent)
    try:   # every TorchTitan model preset of the reference sets model.hf_assets_path; its model-override patch
        # (primus/backends/torchtitan/patches/model_override_patches.py:205-276) raises on any key of the preset that
        # the installed TorchTitan's JobConfig.model does not declare
        import dataclasses
        from torchtitan.config.job_config import JobConfig
        model_t = {f.name: f.type for f in dataclasses.fields(JobConfig)}["model"]
        declared = {f.name for f in dataclasses.fields(model_t)}
    except Exception as e:  # noqa: BLE001
        return _reference_unavailable(f"cannot inspect the installed torchtitan ({type(e).__name__}: {e})")
    if "hf_assets_path" not in declared:
        return _reference_unavailable(
            "reference TorchTitan backend needs a newer torchtitan than the one installed (0.1.0): its stock model "
            "presets set model.hf_assets_path and its model-override patch raises \"'TransformerModelArgs' has no "
            "field 'hf_assets_path'\" (observed on a B200 box); its pinned third_party/torchtitan and "
            "third_party/Megatron-LM submodule directories are empty, Transformer-Engine / Primus-Turbo are not "
            "installed, and pip cannot build the package offline (hatchling is not in the wheelhouse)")
    if not os.path.exists("/dev/nvidiactl"):
        return _reference_unavailable("reference TorchTitan backend needs a GPU")
    work = Path(tempfile.mkdtemp(prefix="primus_ref_"))
    _reference_tokenizer_assets(work / "tokenizer")
    steps = args.warmup + args.steps
    gbs = args.batch_per_gpu * world
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ref) + os.pathsep + env.get("PYTHONPATH", "")
    env.setdefault("RANK", "0"), env.setdefault("LOCAL_RANK", "0"), env.setdefault("WORLD_SIZE", "1")
    env.setdefault("MASTER_ADDR", "127.0.0.1"), env.setdefault("MASTER_PORT", "29533")
    env.setdefault("LOCAL_WORLD_SIZE", env["WORLD_SIZE"])
    last = ""
    for ac_mode in (["selective", "full"] if args.ref_ac == "auto" else [args.ref_ac]):
        cmd = [sys.executable, "-m", "primus.cli.main", "train", "pretrain", "--config", str(cfg),
               "--backend_path", backend_path,
               "--training.mock_data", "true", "--training.steps", str(steps), "--training.seq_len", str(args.seq),
               "--training.local_batch_size", str(args.micro_batch), "--training.global_batch_size", str(gbs),
               "--training.gc_freq", "1000", "--metrics.log_freq", "1", "--lr_scheduler.warmup_steps", "2",
               "--model.tokenizer_path", str(work / "tokenizer"),
               "--activation_checkpoint.mode", ac_mode, "--activation_checkpoint.selective_ac_option", "op",
               "--primus_turbo.enable_primus_turbo", "false"]
        log = work / f"rank{rank}_{ac_mode}.log"
        with open(log, "w") as f:
            rc = subprocess.run(cmd, cwd=work, env=env, stdout=f, stderr=subprocess.STDOUT).returncode
        text = re.sub(r"\x1b\[[0-9;]*m", "", log.read_text(errors="replace"))
        if rank == 0 and args.ref_log:
            Path(args.ref_log).parent.mkdir(parents=True, exist_ok=True)
            Path(args.ref_log).write_text(text[-200000:])
        tps = [float(m.group(2).replace(",", "")) for m in
               re.finditer(r"step:\s*(\d+).*?tps:\s*([\d,\.]+)", text)]
        if rc == 0 and len(tps) >= steps:
            break
        last = " | ".join(l.strip()[-200:] for l in text.splitlines()[-400:] if "Error" in l or "error" in l)[-600:]
        tps = []
    if not tps:
        return _reference_unavailable("reference TorchTitan path failed on this box: " + (last or "no step lines"))
    if rank == 0:
        timed = tps[-args.steps:]
        tokens_rank_step = gbs // world * args.seq
        ms = sum(tokens_rank_step / t * 1e3 for t in timed) / len(timed)
        value = gbs * args.seq / (ms / 1e3)
        print(json.dumps({
            "impl": "reference", "metric": "tokens/s (Llama-3.1-8B pretraining, whole job)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / (BASELINE_TOK_S_GPU * world),
            "dtype": "bf16 (fp32 master parameters, bf16 compute, fp32 gradient reduction)",
            "data": "synthetic: the reference's mock dataset (uniform-random ids below 32000), random-init weights",
            "config": {"model": "llama3.1_8B", "global_batch": gbs, "seq_len": args.seq,
                       "micro_batch": args.micro_batch, "parallelism": f"fsdp{world}",
                       "backend": "reference CLI -> TorchTitan backend, torch.compile on, activation checkpoint "
                                  + ac_mode + ", Primus-Turbo off (not installed)",
                       "timing": "reference's own per-step tps log line (wall clock after the loss read-back)"},
            "tokens_per_s_per_gpu": value / world}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="primus_b200")
    ap.add_argument("--model", default="llama3.1_8B")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--batch-per-gpu", type=int, default=16)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (with sequence parallelism); dp = gpus / tp")
    ap.add_argument("--cp", type=int, default=1, help="context-parallel size; dp = gpus / (tp * cp)")
    ap.add_argument("--cp-comm", default="a2a", choices=["a2a", "allgather", "p2p", "a2a+p2p"],
                    help="context-parallel scheme: all-to-all over heads (Ulysses), K/V all-gather with zig-zag chunks, or ring (p2p)")
    ap.add_argument("--fused-tp", action="store_true", help="fused all-gather->GEMM / GEMM->reduce-scatter kernels")
    ap.add_argument("--fused-dp", dest="fused_dp", action="store_true", default=None,
                    help="fused P2P reduce-scatter (overlapped with backward) + AdamW + all-gather by peer stores "
                         "(default on more than one GPU)")
    ap.add_argument("--no-fused-dp", dest="fused_dp", action="store_false",
                    help="NCCL reduce-scatter / all-gather around the AdamW kernel instead")
    ap.add_argument("--no-overlap-param-gather", action="store_true",
                    help="NCCL path: wait for the parameter all-gather right after the optimizer step")
    ap.add_argument("--grad-reduce", default="bf16", choices=["bf16", "fp32"],
                    help="wire format of the data-parallel gradient reduction (accumulation stays fp32); the reference's "
                         "MXFP8 recipe sets grad_reduce_in_bf16")
    ap.add_argument("--precision", default="mxfp8", choices=["bf16", "mxfp8"],
                    help="linear-layer GEMM precision: bf16, or MXFP8 (E4M3 values, UE8M0 scale per 32 elements; fp32 accumulation)")
    ap.add_argument("--ref-ac", default="auto", choices=["auto", "none", "selective", "full"],
                    help="reference arm: activation checkpointing mode (auto = selective, then full if that fails)")
    ap.add_argument("--ref-log", default=None, help="reference arm: copy rank 0's log of the reference run here")
    ap.add_argument("--mem-fraction", type=float, default=0.0,
                    help="cap this process's device memory (testing the out-of-memory fallback of the warm-up)")
    ap.add_argument("--layers", type=int, default=0,
                    help="truncate the model to this many layers (stated in `config`; never for the headline number)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline-parallel size")
    ap.add_argument("--vpp", type=int, default=0, help="virtual pipeline stages per rank (interleaved schedule)")
    ap.add_argument("--schedule", default=None, help="pipeline schedule: 1f1b | interleaved | zerobubble | zbv | v-half | v-min")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel size (MoE models)")
    ap.add_argument("--fused-ep", action="store_true", help="fused dispatch + GEMM / GEMM + combine kernels (use_turbo_mega_moe)")
    ap.add_argument("--bf16-moments", action="store_true", help="Adam moments in bf16 (precision-aware optimizer)")
    ap.add_argument("--recompute-layers", type=int, default=0, help="full recomputation of the first N layers of every stage")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import _lib
    from primus_b200.parallel import state as ps

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.fused_dp is None:
        args.fused_dp = world > 1 and args.tp * args.cp * args.pp < world and args.ep == 1 and not args.bf16_moments
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        ps.init_distributed("nccl")
    _lib.require()
    warmup = max(args.warmup, 3)

    par = dict(params_dtype="bf16", seq_length=args.seq, tensor_model_parallel_size=args.tp,
               sequence_parallel=args.tp > 1, fp8="e4m3" if args.precision == "mxfp8" else None,
               fp8_recipe="mxfp8", context_parallel_size=args.cp, cp_comm_type=args.cp_comm,
               hierarchical_context_parallel_sizes=[2, args.cp // 2] if args.cp_comm == "a2a+p2p" else None,
               pipeline_model_parallel_size=args.pp, virtual_pipeline_model_parallel_size=args.vpp or None,
               expert_model_parallel_size=args.ep)
    if args.model in MODELS:
        mdict = dict(MODELS[args.model])
    else:       # any model preset of the package (primus_b200/configs/models/<name>.yaml)
        import dataclasses

        from primus_b200.core.config.presets import load_preset

        names = {f.name for f in dataclasses.fields(TransformerConfig)}
        mdict = {k: v for k, v in load_preset(args.model, "models").items() if k in names and k not in par}
    full_layers = mdict["num_layers"]
    if args.layers:
        mdict["num_layers"] = args.layers
        if isinstance(mdict.get("moe_layer_freq"), str) and mdict.get("num_experts"):
            from primus_b200.models.config import parse_moe_layer_freq

            mdict["moe_layer_freq"] = parse_moe_layer_freq(mdict["moe_layer_freq"], full_layers)[:args.layers]
    if args.recompute_layers:
        mdict.update(recompute_granularity="full", recompute_method="block", recompute_num_layers=args.recompute_layers)
    if args.fused_ep:
        mdict["use_turbo_mega_moe"] = True
    mcfg = TransformerConfig(**mdict, **par)
    if args.fused_tp:
        from primus_b200.parallel import fused_tp

        fused_tp.ENABLED = True          # all-gather -> GEMM; the reduce-scatter side stays on NCCL (faster at tp = 8)
    gbs = args.batch_per_gpu * world // (args.tp * args.cp * args.pp)
    schedule = args.schedule or ("interleaved" if args.vpp else "1f1b")
    tcfg = TrainConfig(micro_batch_size=args.micro_batch, global_batch_size=gbs, seq_length=args.seq,
                       train_iters=10 ** 6, lr=3e-4, lr_warmup_iters=100, lr_decay_iters=10 ** 6, weight_decay=0.1,
                       clip_grad=1.0, use_distributed_optimizer=True, overlap_grad_reduce=world > 1,
                       log_interval=10 ** 9, manual_gc=True, fused_dp_optimizer=args.fused_dp,
                       pipeline_schedule=schedule, use_precision_aware_optimizer=args.bf16_moments,
                       exp_avg_dtype="bf16" if args.bf16_moments else "fp32",
                       exp_avg_sq_dtype="bf16" if args.bf16_moments else "fp32",
                       overlap_param_gather=world > 1 and not args.no_overlap_param_gather,
                       grad_reduce_in_bf16=world > 1 and args.grad_reduce == "bf16" and not args.fused_dp)
    ps.initialize_model_parallel(tp=args.tp, pp=args.pp, cp=args.cp, ep=args.ep, virtual_pp=args.vpp or None)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    import gc
    if args.mem_fraction:
        torch.cuda.set_per_process_memory_fraction(args.mem_fraction, local_rank)
    # One GPU holds all optimizer state of the 8B model (the peak is ~174 of 179 GiB): if the warm-up runs out of
    # memory, retry with full activation recomputation of the first 4, 8, then 16 layers and say so in `config`.
    recomputed = 0
    for attempt in range(4):
        trainer = None
        try:
            trainer = Trainer(mcfg, tcfg, device=f"cuda:{local_rank}", log_fn=lambda s: None)
            gc.disable()
            for _ in range(warmup):
                loss = trainer.train_step()
            break
        except torch.OutOfMemoryError:
            gc.enable()
            if world > 1 or attempt == 3:
                raise
            recomputed = 4 << attempt
            print(f"[bench] out of memory during warm-up: retrying with recomputation of {recomputed} layers",
                  file=sys.stderr)
        del trainer
        loss = None
        gc.collect()
        torch.cuda.empty_cache()
        mcfg.recompute_granularity = "full"
        mcfg.recompute_layer_ids = list(range(recomputed))
    barrier()
    _lib.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---------------------------------------------------------------- device-timed region
    launches0 = _lib.LAUNCH_COUNT
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        loss = trainer.train_step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = _lib.LAUNCH_COUNT - launches0
    h2d = trainer.stager.h2d_bytes_last_step
    # ---------------------------------------------------------------- end-to-end region
    e2e_ms = None
    d2h = 0
    if not args.no_e2e:
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev2.record()
        host_losses = []
        for _ in range(args.steps):
            l = trainer.train_step()
            host_losses.append(float(l.item()))  # device -> host read of the step result
            d2h = l.numel() * l.element_size()
        ev3.record()
        barrier()
        e2e_ms = ev2.elapsed_time(ev3)
    clocks = sampler.stop() if rank == 0 else {}
    gc.enable()
    _lib.check_status()

    t = torch.tensor([ms, e2e_ms or 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    tokens_per_step = gbs * args.seq
    value = tokens_per_step * args.steps / (ms / 1e3)
    final_loss = trainer.reduced_loss(loss)
    if rank == 0:
        flops_tok = trainer.flops_per_token
        out = {
            "metric": "tokens/s (Llama-3.1-8B pretraining, whole job)" if args.model == "llama3.1_8B"
            else f"tokens/s ({args.model})",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / (BASELINE_TOK_S_GPU * world) if args.model == "llama3.1_8B" else None,
            "dtype": "bf16" if args.precision == "bf16" else "mxfp8 linear GEMMs (E4M3 + UE8M0 per 32, fp32 accumulate), bf16 attention / LM head / params, fp32 master",
            "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
            "config": {"model": args.model + (f"[truncated to {args.layers} of {full_layers} layers]" if args.layers else ""), "global_batch": gbs, "seq_len": args.seq,
                       "micro_batch": args.micro_batch, "parallelism": f"dp{world // (args.tp * args.cp * args.pp)}" + (f"tp{args.tp}sp" if args.tp > 1 else "") + (f"pp{args.pp}" + (f"vpp{args.vpp}" if args.vpp else "") + f"-{schedule}" if args.pp > 1 else "") + (f"ep{args.ep}" + ("+fused_ep" if args.fused_ep else "") if args.ep > 1 or args.fused_ep else "") + (f"cp{args.cp}-{args.cp_comm}" if args.cp > 1 else "") + ("+fused_tp" if args.fused_tp else "") + ("+fused_dp" if args.fused_dp else ""),
                       "optimizer": "distributed AdamW, fp32 master + fp32 main grads, clip 1.0" + (
                           "" if world == 1 else (", fused P2P reduce-scatter overlapped with backward" if args.fused_dp else
                                                  f", NCCL reduce-scatter in {args.grad_reduce} overlapped with backward, "
                                                  + ("parameter all-gather overlapped with the next forward"
                                                     if not args.no_overlap_param_gather else "blocking parameter all-gather"))),
                       "recompute": f"full recomputation of the first {recomputed} layers (out-of-memory fallback)" if recomputed else (f"full recomputation of the first {args.recompute_layers} layers of every stage" if args.recompute_layers else "none"),
                       "cache": "inputs_larger_than_L2 (per-step working set >> 126 MB)"},
            "tokens_per_s_per_gpu": value / world,
            "model_tflops_per_gpu": value / world * flops_tok / 1e12,
            "gpu_launches": launches, "loss": final_loss, "clocks": clocks,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
            "baseline_ref": "16224 tok/s/GPU, Llama-3.1-8B FP8 on 8x MI325X (reference docs)",
            "impl": "primus_b200",
        }
        if e2e_ms:
            e2e_val = tokens_per_step * args.steps / (e2e_ms / 1e3)
            out["e2e"] = {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                          "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
