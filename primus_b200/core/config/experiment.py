"""Experiment files.

An experiment YAML has the reference's shape
(examples/megatron/configs/MI355X/llama3.1_8B-BF16-pretrain.yaml:1-71, parser
primus/core/launcher/parser.py:192-347):

    work_group: ...          # required meta keys
    user_name: ...
    exp_name: ...
    workspace: ./output
    platform: {config: platform_local.yaml, overrides: {...}}      # optional
    env: {NCCL_DEBUG: WARN}                                        # optional, exported before start-up
    modules:
      pre_trainer:
        framework: megatron            # accepted and ignored: single backend
        config: pre_trainer.yaml       # module preset  (configs/modules)
        model: llama3.1_8B.yaml        # model preset   (configs/models)
        overrides: {train_iters: 10, ...}

``load_experiment`` resolves presets (model and module presets are merged *without* override — a key
defined in both is an error), applies ``overrides:`` and then CLI overrides, and returns an
:class:`Experiment` whose ``modules[name].params`` is the flat parameter dict the trainer consumes.
Only keys containing "trainer" are treated as trainer modules; ``pre_trainer`` and ``post_trainer`` alias
each other when only one is present (primus/core/config/primus_config.py:147-175).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

import yaml

from .merge import deep_merge, merge_without_override
from .presets import load_preset
from .yaml_loader import load_yaml

REQUIRED_META = ("work_group", "user_name", "exp_name", "workspace")
MODULE_ATTRS = ("trainer_class", "stage")  # module-level attributes that overrides must not erase


@dataclass
class ModuleConfig:
    name: str
    framework: str
    config: Optional[str]
    model: Optional[str]
    params: dict
    trainer_class: Optional[str] = None


@dataclass
class Experiment:
    path: str
    meta: dict
    platform: dict
    env: dict
    modules: dict[str, ModuleConfig] = field(default_factory=dict)
    schema_findings: list = field(default_factory=list)   # unknown / misplaced keys (core/config/schema_check.py)

    @property
    def exp_root_path(self) -> str:
        m = self.meta
        return os.path.join(str(m["workspace"]), str(m["work_group"]), str(m["user_name"]), str(m["exp_name"]))

    def module(self, name: str) -> ModuleConfig:
        if name in self.modules:
            return self.modules[name]
        alias = {"pre_trainer": "post_trainer", "post_trainer": "pre_trainer"}.get(name)
        if alias and alias in self.modules:
            return self.modules[alias]
        raise KeyError(f"experiment {self.path} has no module {name!r} (has: {sorted(self.modules)})")

    def export(self) -> dict:
        return {**self.meta, "platform": self.platform, "env": self.env,
                "modules": {n: {"framework": m.framework, "config": m.config, "model": m.model,
                                "trainer_class": m.trainer_class, "params": m.params}
                            for n, m in self.modules.items()}}

    def dump(self, path: str) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        with open(path, "w") as f:
            yaml.safe_dump(self.export(), f, sort_keys=False)


def _resolve_module(name: str, spec: dict) -> ModuleConfig:
    framework = spec.get("framework", "primus_b200")
    params: dict = {}
    trainer_class = spec.get("trainer_class")
    if spec.get("config"):
        mod = load_preset(spec["config"], "modules", framework)
        trainer_class = mod.pop("trainer_class", trainer_class)
        params = mod
    if spec.get("model"):
        model = load_preset(spec["model"], "models", framework)
        # module and model presets live in (mostly) disjoint key spaces: a key defined in both with two
        # different non-null values is an error, except the parallelism / precision keys below where the
        # module preset wins
        for k in set(params) & set(model):
            a, b = params[k], model[k]
            if a is None:
                params[k] = b
            elif b is not None and a != b and k not in _SHARED_KEYS:
                raise KeyError(f"key {k!r} defined with different values in module preset ({a!r}) and "
                               f"model preset ({b!r})")
        params = merge_without_override(params, model, excepts=set(params) & set(model))
    ov = spec.get("overrides") or {}
    trainer_class = ov.pop("trainer_class", trainer_class) if isinstance(ov, dict) else trainer_class
    params = deep_merge(params, ov)
    return ModuleConfig(name, framework, spec.get("config"), spec.get("model"), params, trainer_class)


_SHARED_KEYS = {
    "tensor_model_parallel_size", "pipeline_model_parallel_size", "expert_model_parallel_size",
    "context_parallel_size", "sequence_parallel", "virtual_pipeline_model_parallel_size", "seq_length",
    "max_position_embeddings", "fp8", "fp8_recipe", "recompute_granularity", "recompute_layer_ids",
    "expert_tensor_parallel_size",
}


def load_experiment(path: str, cli_overrides: Optional[dict] = None, module_for_cli: Optional[str] = None) -> Experiment:
    raw = load_yaml(path)
    missing = [k for k in REQUIRED_META if k not in raw]
    if missing:
        raise KeyError(f"{path}: missing required keys {missing}")
    meta = {k: raw[k] for k in REQUIRED_META}
    plat_spec = raw.get("platform") or {}
    platform = load_preset(plat_spec.get("config", "platform_local.yaml"), "platforms")
    platform = deep_merge(platform, plat_spec.get("overrides") or {})
    exp = Experiment(path=str(path), meta=meta, platform=platform, env=dict(raw.get("env") or {}))
    from . import schema_check

    exp.schema_findings = schema_check.check_experiment(raw, cli_overrides)
    for name, spec in (raw.get("modules") or {}).items():
        if "trainer" not in name:
            continue
        exp.modules[name] = _resolve_module(name, dict(spec or {}))
    if cli_overrides:
        targets = [exp.module(module_for_cli)] if module_for_cli else list(exp.modules.values())
        for m in targets:
            m.params = deep_merge(m.params, cli_overrides)
    return exp


def apply_env_block(exp: Experiment, environ=None) -> dict:
    """Export the experiment's top-level ``env:`` block (values stringified); returns what was set."""
    environ = os.environ if environ is None else environ
    done = {}
    for k, v in exp.env.items():
        environ[str(k)] = "" if v is None else str(v)
        done[str(k)] = environ[str(k)]
    return done
