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
EXTRA_KNOWN = {"trainer_class", "tp_comm_overlap", "tp_comm_overlap_rs", "pp_algorithm", "stage", "framework", "disable_wandb",
               "disable_tensorboard", "disable_mlflow", "valid_data_path"}


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
    return findings
