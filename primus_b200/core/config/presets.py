"""Preset lookup: ``primus_b200/configs/<modules|models|platforms>/<name>.yaml`` with a path-traversal
guard (primus/core/config/preset_loader.py:15-61 in the reference; the ``<framework>`` directory level of
the reference collapses because this framework has a single backend, but a ``framework/name`` form such as
``megatron/llama3_8B.yaml`` is still accepted so that reference experiment files load unchanged)."""
from __future__ import annotations

from pathlib import Path

from .yaml_loader import load_yaml

CONFIG_ROOT = Path(__file__).resolve().parent.parent.parent / "configs"


def preset_path(name: str, kind: str, framework: str | None = None) -> Path:
    if kind not in ("modules", "models", "platforms", "hardware"):
        raise ValueError(f"unknown preset kind {kind!r}")
    base = (CONFIG_ROOT / kind).resolve()
    if not name.endswith((".yaml", ".yml")):
        name += ".yaml"
    cands = [base / name]
    if framework:
        cands.append(base / framework / name)
    cands.append(base / Path(name).name)
    for c in cands:
        c = c.resolve()
        if base not in c.parents and c != base:
            raise ValueError(f"preset {name!r} escapes {base}")
        if c.exists():
            return c
    raise FileNotFoundError(f"no {kind} preset named {name!r} under {base}")


def load_preset(name: str, kind: str, framework: str | None = None) -> dict:
    return load_yaml(preset_path(name, kind, framework))
