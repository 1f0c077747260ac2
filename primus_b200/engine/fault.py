"""Failure detection and recovery on the host side.

* :class:`RerunStateMachine` — result validation by re-execution with host-side error injection
  (``rerun_mode``: disabled | validate_results | report_stats; ``error_injection_rate`` /
  ``error_injection_type``: correct_result | transient_error | persistent_error;
  primus/configs/modules/megatron/trainer_base.yaml:349-352 in the reference).  A step whose loss is not finite
  (or is perturbed by the injector) is recomputed from the same inputs: a different second result classifies the
  fault as *transient* (continue with the recomputed value), the same bad result as *persistent* (stop and
  checkpoint), an identical finite result as a *correct result* (false alarm).
* :class:`LossGuard` — non-finite, spiky-loss and large-gradient checks
  (``check_for_nan_in_loss_and_grad``, ``check_for_spiky_loss``, ``check_for_large_grads``, :22-24).
* :class:`GracefulExit` — SIGTERM / SIGINT set a flag that the training loop polls between steps so that it can
  checkpoint and leave (``exit_signal_handler``, :26-28).
* :class:`StragglerDetector` — per-rank step times exchanged on the host; reports ranks slower than the median
  by a factor (``log_straggler``, :413-416).
* :class:`Heartbeat` — liveness through the rendezvous store: a rank that stops beating is reported by the others
  before their next collective instead of hanging in it.

Nothing here faults, traps or hangs a GPU: injected errors perturb a host copy of the loss, and a lost rank is
detected on the host (store / heartbeat) between steps.
"""
from __future__ import annotations

import math
import random
import signal
import statistics
import time
from dataclasses import dataclass, field
from typing import Callable, Optional


class PersistentFault(RuntimeError):
    pass


@dataclass
class RerunStateMachine:
    mode: str = "disabled"
    error_injection_rate: float = 0.0          # probability per validated step
    error_injection_type: str = "transient_error"
    seed: int = 0
    stats: dict = field(default_factory=lambda: {"validated": 0, "transient": 0, "persistent": 0, "correct": 0,
                                                 "injected": 0})

    def __post_init__(self):
        if self.mode not in ("disabled", "validate_results", "report_stats"):
            raise ValueError(f"unknown rerun_mode {self.mode!r}")
        if self.error_injection_type not in ("correct_result", "transient_error", "persistent_error"):
            raise ValueError(f"unknown error_injection_type {self.error_injection_type!r}")
        self._rng = random.Random(self.seed)
        self._persist = False

    def _inject(self, value: float, attempt: int) -> float:
        """Host-side perturbation of the observed result."""
        t = self.error_injection_type
        if t == "correct_result":
            return value                      # flags the step as suspicious without changing the value
        if t == "transient_error":
            return float("nan") if attempt == 0 else value
        return float("nan")                   # persistent: every attempt is bad

    def run(self, compute: Callable[[], float]) -> float:
        """``compute`` evaluates the step result (loss) deterministically from saved inputs."""
        if self.mode == "disabled":
            return compute()
        first = compute()
        suspicious = not math.isfinite(first)
        injected = self.error_injection_rate > 0 and self._rng.random() < self.error_injection_rate
        if injected:
            self.stats["injected"] += 1
            first = self._inject(first, 0)
            suspicious = True
        if not suspicious:
            return first
        self.stats["validated"] += 1
        second = compute()
        if injected:
            second = self._inject(second, 1)
        same = (first == second) or (math.isnan(first) and math.isnan(second))
        if same and math.isfinite(second):
            self.stats["correct"] += 1
            return second
        if not same and math.isfinite(second):
            self.stats["transient"] += 1
            return second
        self.stats["persistent"] += 1
        if self.mode == "validate_results":
            raise PersistentFault(f"step result is reproducibly invalid ({first!r}, {second!r})")
        return second


@dataclass
class LossGuard:
    check_nan: bool = True
    check_spiky: bool = False
    spike_factor: float = 10.0
    check_large_grads: bool = False
    grad_norm_limit: float = 1e4
    history: list = field(default_factory=list)

    def check(self, loss: float, grad_norm: Optional[float] = None) -> Optional[str]:
        """Returns a description of the problem, or None."""
        if self.check_nan and not math.isfinite(loss):
            return f"non-finite loss {loss!r}"
        if self.check_nan and grad_norm is not None and not math.isfinite(grad_norm):
            return f"non-finite gradient norm {grad_norm!r}"
        if self.check_spiky and len(self.history) >= 4:
            base = statistics.median(self.history[-16:])
            if loss > self.spike_factor * base:
                return f"loss spike: {loss:.4g} vs running median {base:.4g}"
        if self.check_large_grads and grad_norm is not None and grad_norm > self.grad_norm_limit:
            return f"gradient norm {grad_norm:.4g} above limit {self.grad_norm_limit:.4g}"
        self.history.append(loss)
        return None


class GracefulExit:
    def __init__(self, signals=(signal.SIGTERM, signal.SIGINT)):
        self.requested = False
        self.signum = None
        self._old = {}
        for s in signals:
            try:
                self._old[s] = signal.signal(s, self._handler)
            except ValueError:  # not in the main thread
                pass

    def _handler(self, signum, frame):
        self.requested = True
        self.signum = signum

    def restore(self):
        for s, h in self._old.items():
            signal.signal(s, h)


class StragglerDetector:
    def __init__(self, factor: float = 1.3, group=None):
        self.factor, self.group = factor, group
        self.times: list[float] = []

    def record(self, seconds: float):
        self.times.append(seconds)

    def report(self) -> dict:
        """Exchange the mean step time of every rank on the host; returns slow ranks relative to the median."""
        import torch.distributed as dist

        mine = sum(self.times) / max(len(self.times), 1)
        self.times.clear()
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return {"mean_s": [mine], "stragglers": []}
        allv = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(allv, mine, group=self.group)
        med = statistics.median(allv)
        return {"mean_s": allv, "median_s": med,
                "stragglers": [r for r, v in enumerate(allv) if med > 0 and v > self.factor * med]}


class Heartbeat:
    """Rank liveness through a key-value store (``torch.distributed`` TCPStore / FileStore)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s

    def beat(self, step: int):
        self.store.set(f"hb/{self.rank}", f"{step}:{time.time()}")

    def dead_ranks(self, now: Optional[float] = None) -> list[int]:
        now = time.time() if now is None else now
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"hb/{r}").decode()
                _, ts = v.split(":")
                if now - float(ts) > self.timeout_s:
                    dead.append(r)
            except Exception:  # noqa: BLE001  (missing key: never started)
                dead.append(r)
        return dead
