"""Runtime orchestration: configuration -> environment -> distributed context -> logging -> trainer
-> lifecycle with patch phases.

Lifecycle (same order as the reference's ``PrimusRuntime``, primus/core/runtime/train_runtime.py:95-116,
204-229,500-544):  ``build_args`` patches -> trainer constructed -> ``setup`` patches -> ``trainer.setup()``
-> ``trainer.init()`` -> ``before_train`` patches -> ``trainer.train()`` (Python GC disabled) ->
``after_train`` patches -> ``trainer.cleanup()``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Optional

from ..config.experiment import Experiment, apply_env_block, load_experiment
from ..config.overrides import parse_cli_overrides
from ..patches import builtin  # noqa: F401  (registers the built-in patches)
from ..patches.registry import PatchContext, run_patches
from ..utils import env as env_utils
from ..utils import logger as logutil


@dataclass
class RuntimeState:
    """Mutable per-iteration metrics that patches and trainers publish
    (primus/core/runtime/runtime_state.py:20-34)."""
    metrics: dict = field(default_factory=dict)

    def update_metrics(self, **kw):
        self.metrics.update(kw)


@dataclass
class TrainContext:
    experiment: Optional[Experiment] = None
    module_name: str = "pre_trainer"
    params: dict = field(default_factory=dict)
    trainer: Any = None
    state: RuntimeState = field(default_factory=RuntimeState)
    dist_env: dict = field(default_factory=dict)


TRAINER_CLASSES: dict[str, str] = {
    "PretrainTrainer": "primus_b200.engine.pretrain:PretrainTrainer",
    "SFTTrainer": "primus_b200.engine.sft:SFTTrainer",
}


def load_trainer_class(name: str):
    import importlib

    target = TRAINER_CLASSES.get(name, name)
    if ":" not in target:
        raise KeyError(f"unknown trainer class {name!r}; known: {sorted(TRAINER_CLASSES)}")
    mod, cls = target.split(":")
    return getattr(importlib.import_module(mod), cls)


class PrimusRuntime:
    def __init__(self, config_path: str, overrides: Optional[list[str]] = None, export_config: Optional[str] = None):
        self.config_path = config_path
        self.cli_overrides = parse_cli_overrides(overrides or [])
        self.export_config = export_config
        self.ctx = TrainContext()

    # ------------------------------------------------------------------ phases
    def _initialize_configuration(self, module_name: str):
        exp = load_experiment(self.config_path, self.cli_overrides, module_name)
        self.ctx.experiment = exp
        self.ctx.module_name = module_name
        self.ctx.params = exp.module(module_name).params
        apply_env_block(exp)
        for finding in exp.schema_findings:   # typos must not turn into silently ignored settings
            print(f"[primus_b200][config][WARNING] {finding}", flush=True)
        if os.environ.get("PRIMUS_STRICT_CONFIG", "0") == "1" and exp.schema_findings:
            raise KeyError("unknown configuration keys: " + "; ".join(exp.schema_findings))
        if self.export_config:
            exp.dump(self.export_config)

    def _initialize_environment(self):
        exp = self.ctx.experiment
        self.ctx.dist_env = env_utils.get_torchrun_env()
        env_utils.setup_training_env(exp.exp_root_path)
        os.makedirs(exp.exp_root_path, exist_ok=True)
        p = self.ctx.params
        logutil.setup_logger(exp.exp_root_path, self.ctx.module_name, self.ctx.dist_env["rank"],
                             self.ctx.dist_env["world_size"], str(p.get("stderr_sink_level", "INFO")),
                             str(p.get("file_sink_level", "DEBUG")))

    def _initialize_trainer(self):
        exp = self.ctx.experiment
        pctx = PatchContext(phase="build_args", params=self.ctx.params, experiment=exp,
                            extra={"exp_root_path": exp.exp_root_path})
        run_patches("build_args", pctx, log=logutil.get_logger().debug)
        mod = exp.module(self.ctx.module_name)
        cls = load_trainer_class(mod.trainer_class or self.ctx.params.get("trainer_class") or "PretrainTrainer")
        self.ctx.trainer = cls(self.ctx.params, exp, self.ctx.state)
        return self.ctx.trainer

    def _run_trainer_lifecycle(self):
        import gc

        tr = self.ctx.trainer
        exp = self.ctx.experiment
        mk = lambda ph: PatchContext(phase=ph, params=self.ctx.params, trainer=tr, experiment=exp,  # noqa: E731
                                     extra={"exp_root_path": exp.exp_root_path})
        run_patches("setup", mk("setup"))
        tr.setup()
        tr.init()
        run_patches("before_train", mk("before_train"))
        gc_was = gc.isenabled()
        gc.disable()
        try:
            tr.train()
        finally:
            if gc_was:
                gc.enable()
        run_patches("after_train", mk("after_train"))
        tr.cleanup()

    # ------------------------------------------------------------------ public API
    def run_train_module(self, module_name: str = "pre_trainer"):
        self._initialize_configuration(module_name)
        self._initialize_environment()
        self._initialize_trainer()
        self._run_trainer_lifecycle()
        return self.ctx

    def setup_model_only(self, module_name: str = "pre_trainer"):
        """Build configuration and trainer (model + optimizer) without training: used by the projection
        tool's benchmark mode (primus/core/runtime/train_runtime.py:118-176)."""
        self._initialize_configuration(module_name)
        self._initialize_environment()
        tr = self._initialize_trainer()
        tr.setup()
        tr.init()
        return tr
