"""Static check of experiment configs: unknown or misplaced keys.

A key given in a module's ``overrides:`` block (or on the command line) is *known* when it is a field of the
engine's ``TransformerConfig`` / ``TrainConfig`` or appears in the module / model preset the module is built
from (presets also carry keys that only the launcher, logging or optional features consume).  Anything else is
reported with the closest known names, which catches the typos that otherwise turn into silently ignored
settings.  Role of the reference's schema check (primus/core/config/schema_check.py), which compares against the
backend's argument namespace; here the namespace is the two dataclasses plus the presets.
"""
from __future__ import annotations

import dataclasses
import difflib
from typing import Iterable

from .presets import load_preset

# keys consumed outside the two config dataclasses (launcher, patches, logging, optional features)
EXTRA_KNOWN = {"train_samples", "lr_warmup_samples", "lr_decay_samples", "trainer_class", "tp_comm_overlap", "tp_comm_overlap_rs", "pp_algorithm", "stage", "framework", "disable_wandb",
               "disable_tensorboard", "disable_mlflow", "valid_data_path"}


# Keys the presets carry for compatibility with the reference's configuration surface but that this engine does not
# act on.  Setting one of them to something other than the preset's value is reported (an error under
# PRIMUS_STRICT_CONFIG=1), so that no setting is accepted and then silently ignored.  tests/test_config_cpu.py checks
# that every preset key is either read by the code base or listed here.
INERT_KEYS = {
    # numerics fixed by the design: bf16 parameters, fp32 main gradients and accumulation, no loss scaling
    "accumulate_allreduce_grads_in_fp32", "loss_scale", "ddp_average_in_collective",
    # model switches of architectures that are not built (biases, LayerNorm, learned positions)
    "normalization", "position_embedding_type",
    # adapters are folded into the effective weight before the forward pass: there is no separate adapter input to drop
    "lora_dropout",
    # the trainer stages its own batches (sequential sample order; attention masks come from the kernels)
    "create_attention_mask_in_dataloader", "dataloader_type",
    # kernel selection switches of the reference's operator library: one native implementation here
    "cross_entropy_fusion_impl", "use_turbo_attention", "use_turbo_parallel_linear",
    "use_turbo_rms_norm", "turbo_deepep_num_cu", "use_turbo_deepep", "use_turbo_grouped_gemm",
    "use_turbo_fused_act_with_probs", "moe_permute_fusion", "moe_router_padding_for_quantization",
    # the profiler is torch.profiler whenever ``profile`` is set
    "use_pytorch_profiler",
    # services that are not built
    "enable_ft_package", "enable_gloo_process_groups", "straggler_ctrlr_port",
    "trainable",
    "offload_ops",
    # switches between the reference's two pipeline implementations (one runtime here; the schedule is chosen with
    # pp_algorithm / pipeline_schedule or enable_zero_bubble + zero_bubble_v_schedule)
    "patch_primus_pipeline", "patch_zero_bubble", "pp_communication_method",
}


def known_keys(module_preset: str | None = None, model_preset: str | None = None, framework: str = "primus_b200") -> set:
    from ...engine.trainer import TrainConfig
    from ...models.config import TransformerConfig

    keys = {f.name for f in dataclasses.fields(TransformerConfig)} | {f.name for f in dataclasses.fields(TrainConfig)}
    keys |= EXTRA_KNOWN
    if module_preset:
        keys |= set(load_preset(module_preset, "modules", framework))
    if model_preset:
        keys |= set(load_preset(model_preset, "models", framework))
    return keys


def check_keys(given: Iterable[str], known: set) -> list[dict]:
    """One record per unknown key: ``{"key", "suggestions"}``."""
    out = []
    for k in given:
        if k not in known:
            out.append({"key": k, "suggestions": difflib.get_close_matches(k, known, n=3, cutoff=0.75)})
    return out


def check_experiment(raw: dict, cli_overrides: dict | None = None) -> list[str]:
    """Human-readable findings for a loaded experiment YAML (the dict before preset resolution)."""
    findings = []
    for name, spec in (raw.get("modules") or {}).items():
        if "trainer" not in name or not isinstance(spec, dict):
            continue
        known = known_keys(spec.get("config"), spec.get("model"), spec.get("framework", "primus_b200"))
        given = list((spec.get("overrides") or {}).keys()) + list((cli_overrides or {}).keys())
        for rec in check_keys(given, known):
            hint = f" (did you mean {', '.join(rec['suggestions'])}?)" if rec["suggestions"] else ""
            findings.append(f"modules.{name}: unknown key {rec['key']!r}{hint}")
        findings += [f"modules.{name}: {msg}" for msg in
                     check_inert({**(spec.get("overrides") or {}), **(cli_overrides or {})},
                                 spec.get("config"), spec.get("model"), spec.get("framework", "primus_b200"))]
    return findings


def check_inert(values: dict, module_preset: str | None = None, model_preset: str | None = None,
                framework: str = "primus_b200") -> list[str]:
    """Settings that parse but change nothing: a key of ``INERT_KEYS`` given a value other than its preset default."""
    defaults: dict = {}
    if module_preset:
        defaults.update(load_preset(module_preset, "modules", framework))
    if model_preset:
        defaults.update(load_preset(model_preset, "models", framework))
    out = []
    for k, v in values.items():
        if k in INERT_KEYS and k in defaults and v != defaults[k]:
            out.append(f"key {k!r} = {v!r} is accepted for compatibility but has no effect in this engine "
                       f"(preset value {defaults[k]!r})")
        elif k in INERT_KEYS and k not in defaults and v not in (None, False, 0):
            out.append(f"key {k!r} = {v!r} is accepted for compatibility but has no effect in this engine")
    return out
