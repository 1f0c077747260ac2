"""YAML loading with environment substitution and ``extends:`` inheritance.

* ``${VAR}`` must be set (``KeyError`` otherwise); ``${VAR:default}`` falls back to the default.  When a
  scalar consists of exactly one substitution the result is coerced to bool / int / float / null;
  text with a substitution embedded in it stays a string.  Values without substitutions keep the type
  the YAML parser gave them.
* ``extends:`` (a path or a list of paths, relative to the including file) names base files that are
  deep-merged in order; keys of the including file win.

Behavioural parity: primus/core/config/yaml_loader.py:51-128 (substitution), :134-169 (extends).
"""
from __future__ import annotations

import os
import re
from pathlib import Path
from typing import Any

import yaml

from .merge import deep_merge

_VAR = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)(?::([^}]*))?\}")


def _coerce(text: str) -> Any:
    low = text.strip().lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("null", "none", "~", ""):
        return None if low != "" else ""
    try:
        return int(text)
    except ValueError:
        pass
    try:
        return float(text)
    except ValueError:
        return text


def substitute_env(value: Any, env=None) -> Any:
    """Recursively substitute ``${VAR}`` / ``${VAR:default}`` in strings of a parsed YAML tree."""
    env = os.environ if env is None else env
    if isinstance(value, dict):
        return {k: substitute_env(v, env) for k, v in value.items()}
    if isinstance(value, list):
        return [substitute_env(v, env) for v in value]
    if not isinstance(value, str) or "${" not in value:
        return value

    def repl(m: re.Match) -> str:
        name, default = m.group(1), m.group(2)
        if name in env:
            return str(env[name])
        if default is not None:
            return default
        raise KeyError(f"environment variable {name} is required by the config but not set")

    whole = _VAR.fullmatch(value.strip())
    out = _VAR.sub(repl, value)
    return _coerce(out) if whole else out


def load_yaml(path: str | os.PathLike, _stack: tuple = ()) -> dict:
    """Load one YAML file with substitution and ``extends`` resolution."""
    p = Path(path).resolve()
    if p in _stack:
        raise ValueError("cyclic extends: " + " -> ".join(str(s) for s in _stack + (p,)))
    with open(p) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ValueError(f"{p}: top level of a config file must be a mapping")
    data = substitute_env(data)
    bases = data.pop("extends", None)
    if bases is None:
        return data
    if isinstance(bases, str):
        bases = [bases]
    merged: dict = {}
    for b in bases:
        bp = Path(b)
        if not bp.is_absolute():
            bp = p.parent / bp
        merged = deep_merge(merged, load_yaml(bp, _stack + (p,)))
    return deep_merge(merged, data)
