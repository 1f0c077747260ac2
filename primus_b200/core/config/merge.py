"""Dictionary / namespace merge helpers (primus/core/config/merge_utils.py:11-60,
primus/core/utils/yaml_utils.py:19-154 in the reference)."""
from __future__ import annotations

import copy
from types import SimpleNamespace
from typing import Any


def deep_merge(base: dict, override: dict) -> dict:
    """New dict: ``override`` wins; nested dicts merge recursively; other values are replaced."""
    out = copy.deepcopy(base)
    for k, v in override.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def shallow_merge(base: dict, override: dict) -> dict:
    out = dict(base)
    out.update(override)
    return out


def merge_without_override(dst: dict, src: dict, excepts=()) -> dict:
    """Add keys of ``src`` that ``dst`` lacks; a key present in both is an error unless listed in
    ``excepts`` (model and module presets must not silently shadow each other)."""
    out = dict(dst)
    for k, v in src.items():
        if k in out and k not in excepts:
            raise KeyError(f"key {k!r} defined twice while merging presets")
        out.setdefault(k, v)
    return out


def dict_to_namespace(d: Any) -> Any:
    if isinstance(d, dict):
        return SimpleNamespace(**{k: dict_to_namespace(v) for k, v in d.items()})
    if isinstance(d, list):
        return [dict_to_namespace(v) for v in d]
    return d


def namespace_to_dict(ns: Any) -> Any:
    if isinstance(ns, SimpleNamespace):
        return {k: namespace_to_dict(v) for k, v in vars(ns).items()}
    if isinstance(ns, list):
        return [namespace_to_dict(v) for v in ns]
    return ns


def set_nested(d: dict, dotted: str, value: Any) -> None:
    keys = dotted.split(".")
    cur = d
    for k in keys[:-1]:
        nxt = cur.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            cur[k] = nxt
        cur = nxt
    cur[keys[-1]] = value
