"""Phase-aware patch (plug-in) registry.

A *patch* is a function ``fn(ctx)`` registered with an id, a phase, a priority and an optional
condition; ``run_patches(phase, ctx)`` applies every matching patch in priority order.  This is
the extension mechanism the reference drives its ~115 backend patches with
(primus/core/patches/patch_registry.py:29-207, patch_runner.py:26-148, context.py:25-79).  In this
single-backend framework patches mutate the resolved parameter dict (``build_args``) or hook the
trainer (``setup`` / ``before_train`` / ``after_train``) instead of monkey-patching third-party code.

``PRIMUS_PATCHES`` selects patches: ``all`` (default), ``none``, or a comma-separated id list.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

PHASES = ("setup", "build_args", "before_train", "after_train", "convert")


@dataclass
class PatchContext:
    phase: str
    backend: str = "primus_b200"
    params: Optional[dict] = None  # resolved module parameters (mutable)
    trainer: Any = None
    experiment: Any = None
    extra: dict = field(default_factory=dict)
    backend_version: Optional[str] = None
    primus_version: Optional[str] = None

    def get_param(self, name: str, default=None):
        if self.params is None:
            return default
        cur: Any = self.params
        for k in name.split("."):
            if not isinstance(cur, dict) or k not in cur:
                return default
            cur = cur[k]
        return cur


@dataclass
class FunctionPatch:
    id: str
    fn: Callable[[PatchContext], Any]
    phase: str
    backend: str = "*"
    priority: int = 50
    condition: Optional[Callable[[PatchContext], bool]] = None
    backend_versions: Optional[str] = None
    primus_versions: Optional[str] = None
    description: str = ""
    tags: tuple = ()

    def applies_to(self, ctx: PatchContext) -> bool:
        if self.phase != ctx.phase:
            return False
        if self.backend not in ("*", ctx.backend):
            return False
        if self.backend_versions and ctx.backend_version and not version_in_range(ctx.backend_version, self.backend_versions):
            return False
        if self.primus_versions and ctx.primus_version and not version_in_range(ctx.primus_version, self.primus_versions):
            return False
        if self.condition is not None and not self.condition(ctx):
            return False
        return True


class PatchRegistry:
    def __init__(self):
        self._by_phase: dict[str, dict[str, list[FunctionPatch]]] = {}
        self._ids: dict[str, FunctionPatch] = {}

    def register(self, patch: FunctionPatch) -> FunctionPatch:
        if patch.phase not in PHASES:
            raise ValueError(f"unknown phase {patch.phase!r}; valid: {PHASES}")
        if patch.id in self._ids:
            raise ValueError(f"patch id {patch.id!r} registered twice")
        self._ids[patch.id] = patch
        self._by_phase.setdefault(patch.backend, {}).setdefault(patch.phase, []).append(patch)
        return patch

    def unregister(self, patch_id: str) -> None:
        p = self._ids.pop(patch_id)
        self._by_phase[p.backend][p.phase].remove(p)

    def get(self, patch_id: str) -> FunctionPatch:
        return self._ids[patch_id]

    def candidates(self, backend: str, phase: str) -> list[FunctionPatch]:
        out = []
        for b in (backend, "*"):
            out.extend(self._by_phase.get(b, {}).get(phase, []))
        return sorted(out, key=lambda p: (p.priority, p.id))

    def ids(self) -> list[str]:
        return sorted(self._ids)

    def clear(self) -> None:
        self._by_phase.clear()
        self._ids.clear()


REGISTRY = PatchRegistry()


def register_patch(id: str, phase: str, backend: str = "*", priority: int = 50, condition=None,
                   backend_versions: Optional[str] = None, primus_versions: Optional[str] = None,
                   description: str = "", tags: tuple = (), registry: Optional[PatchRegistry] = None):
    """Decorator form: ``@register_patch("args.mock_data", phase="build_args")``."""

    def deco(fn):
        (registry or REGISTRY).register(FunctionPatch(id, fn, phase, backend, priority, condition, backend_versions,
                                                      primus_versions, description or (fn.__doc__ or "").strip(), tags))
        return fn

    return deco


def _selected(env_value: Optional[str]):
    v = (env_value or "all").strip()
    if v.lower() == "all":
        return None
    if v.lower() == "none":
        return set()
    return {x.strip() for x in v.split(",") if x.strip()}


def run_patches(phase: str, ctx: Optional[PatchContext] = None, registry: Optional[PatchRegistry] = None,
                dry_run: bool = False, stop_on_error: bool = True, log: Callable[[str], None] = lambda s: None) -> list[str]:
    """Apply the patches of a phase; returns the ids applied (or that would be, with ``dry_run``)."""
    ctx = ctx or PatchContext(phase=phase)
    ctx.phase = phase
    reg = registry or REGISTRY
    chosen = _selected(os.environ.get("PRIMUS_PATCHES"))
    applied = []
    for p in reg.candidates(ctx.backend, phase):
        if chosen is not None and p.id not in chosen:
            continue
        if not p.applies_to(ctx):
            continue
        applied.append(p.id)
        if dry_run:
            log(f"[patch:{phase}] would apply {p.id}")
            continue
        try:
            p.fn(ctx)
            log(f"[patch:{phase}] applied {p.id}")
        except Exception as e:  # noqa: BLE001
            log(f"[patch:{phase}] {p.id} failed: {e}")
            if stop_on_error:
                raise
    return applied


# ---- semantic-version ranges such as ">=0.8,<0.12" or "==1.2.*"
def _ver(s: str) -> tuple:
    return tuple(int(x) for x in re.findall(r"\d+", s)[:3]) or (0,)


def version_in_range(version: str, spec: str) -> bool:
    v = _ver(version)
    for part in spec.split(","):
        part = part.strip()
        if not part:
            continue
        m = re.match(r"(>=|<=|==|!=|>|<)?\s*(.+)", part)
        op, rhs = m.group(1) or "==", m.group(2)
        if rhs.endswith(".*"):
            pref = _ver(rhs[:-2])
            ok = v[:len(pref)] == pref
            if (op == "==" and not ok) or (op == "!=" and ok):
                return False
            continue
        r = _ver(rhs)
        n = max(len(v), len(r))
        a, b = v + (0,) * (n - len(v)), r + (0,) * (n - len(r))
        if not {"==": a == b, "!=": a != b, ">=": a >= b, "<=": a <= b, ">": a > b, "<": a < b}[op]:
            return False
    return True
