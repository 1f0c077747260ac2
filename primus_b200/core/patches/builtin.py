"""Built-in ``build_args`` patches: the normalisations the reference applies to the resolved arguments
before the trainer is built (primus/backends/megatron/patches/args/*.py,
primus/backends/megatron/patches/args/rocm_arg_validation.py)."""
from __future__ import annotations

import os

from ...models.config import parse_moe_layer_freq
from .registry import PatchContext, register_patch


@register_patch("args.checkpoint_path", phase="build_args", priority=10)
def _checkpoint_paths(ctx: PatchContext):
    """``save`` / ``load`` default to ``<exp_root>/checkpoints``."""
    root = ctx.extra.get("exp_root_path")
    if not root:
        return
    p = ctx.params
    if p.get("save") is None and p.get("save_interval"):
        p["save"] = os.path.join(root, "checkpoints")
    if p.get("load") is None and p.get("auto_continue_train"):
        cand = os.path.join(root, "checkpoints")
        if os.path.exists(os.path.join(cand, "latest_checkpointed_iteration.txt")):
            p["load"] = cand


@register_patch("args.tensorboard_path", phase="build_args", priority=10)
def _tensorboard_path(ctx: PatchContext):
    root = ctx.extra.get("exp_root_path")
    if root and not ctx.params.get("disable_tensorboard", True) and not ctx.params.get("tensorboard_dir"):
        ctx.params["tensorboard_dir"] = os.path.join(root, "tensorboard")


@register_patch("args.mock_data", phase="build_args", priority=20)
def _mock_data(ctx: PatchContext):
    """Mock data needs no tokenizer: NullTokenizer and a default vocabulary."""
    p = ctx.params
    if p.get("mock_data"):
        p["tokenizer_type"] = "NullTokenizer"
        if not p.get("vocab_size"):
            p["vocab_size"] = 131072
        p["data_path"] = None


@register_patch("args.data_path_split", phase="build_args", priority=20)
def _data_path_split(ctx: PatchContext):
    """A space-separated ``data_path`` string becomes a list."""
    for k in ("data_path", "train_data_path", "valid_data_path", "test_data_path"):
        v = ctx.params.get(k)
        if isinstance(v, str) and " " in v.strip():
            ctx.params[k] = v.split()


@register_patch("args.moe_layer_freq", phase="build_args", priority=20)
def _moe_layer_freq(ctx: PatchContext):
    p = ctx.params
    if p.get("num_experts") and isinstance(p.get("moe_layer_freq"), str) and p.get("num_layers"):
        p["moe_layer_freq"] = parse_moe_layer_freq(p["moe_layer_freq"], p["num_layers"])


@register_patch("args.sequence_parallel_tp1", phase="build_args", priority=30)
def _sp_tp1(ctx: PatchContext):
    """Sequence parallelism is meaningless without tensor parallelism."""
    if ctx.params.get("tensor_model_parallel_size", 1) == 1:
        ctx.params["sequence_parallel"] = False


@register_patch("args.iterations_to_skip_default", phase="build_args", priority=30)
def _iters_to_skip(ctx: PatchContext):
    ctx.params.setdefault("iterations_to_skip", [])


@register_patch("args.validate", phase="build_args", priority=90)
def _validate(ctx: PatchContext):
    p = ctx.params
    stage = p.get("turbo_sync_free_moe_stage", 0) or 0
    if stage:
        if not p.get("enable_primus_turbo", True):
            raise ValueError("turbo_sync_free_moe_stage needs enable_primus_turbo")
        p["moe_permute_fusion"] = True
        if stage >= 2:
            p["use_turbo_grouped_gemm"] = True
        if stage >= 3:
            p["use_turbo_fused_act_with_probs"] = True
        if p.get("fp8") or p.get("fp4"):
            p["moe_router_padding_for_quantization"] = True
    if p.get("use_turbo_mega_moe"):
        ep = p.get("expert_model_parallel_size", 1)
        if not (1 < ep <= 8):
            raise ValueError("use_turbo_mega_moe needs 1 < expert_model_parallel_size <= 8 "
                             "(the fused all-to-all rides intra-node peer memory)")
    if p.get("fp8") and p.get("fp8_recipe", "mxfp8") not in ("tensorwise", "blockwise", "mxfp8", "delayed"):
        raise ValueError("fp8 GEMMs support recipes delayed | tensorwise | blockwise | mxfp8")
    if p.get("fp4") and p.get("fp4_recipe", "mxfp4") != "mxfp4":
        raise ValueError("fp4 GEMMs support the mxfp4 recipe only")
    if p.get("use_turbo_autotune") and not p.get("deterministic_mode"):
        # online tile tuning of the tcgen05 GEMMs: each new shape times its candidates once (ops/autotune.py)
        os.environ["PRIMUS_B200_AUTOTUNE"] = "1"
        from ...ops import autotune

        autotune.set_online(True)
    if p.get("deterministic_mode"):
        os.environ.setdefault("PRIMUS_DETERMINISTIC", "1")
        os.environ.setdefault("NCCL_ALGO", "Ring")
    etp = p.get("expert_tensor_parallel_size") or 1
    if etp != 1:
        raise ValueError("expert_tensor_parallel_size > 1 is not supported")
