"""Named step timers in the style of Megatron's ``timers`` (``timing_log_level`` 0 / 1 / 2, ``timing_log_option``
max | minmax | all; primus/configs/modules/megatron/trainer_base.yaml:322-323).

On a GPU a timer brackets its region with CUDA events on the current stream, so starting and stopping never
synchronises; elapsed times are read (one synchronise) only when the log line is written.  On CPU it uses the wall
clock.  ``log`` reduces over the ranks of the job and returns the line Megatron prints:
``(min, max) time across ranks (ms):`` followed by one row per timer.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


class _Timer:
    def __init__(self, name: str, cuda: bool):
        self.name, self.cuda = name, cuda
        self.pairs = []          # finished (start, stop) event pairs, or wall-clock durations
        self._start = None

    def start(self):
        if self.cuda:
            self._start = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._start = time.perf_counter()

    def stop(self):
        if self._start is None:
            return
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.pairs.append((self._start, e))
        else:
            self.pairs.append(time.perf_counter() - self._start)
        self._start = None

    def elapsed_ms(self, reset: bool = True) -> float:
        if self.cuda:
            if self.pairs:
                self.pairs[-1][1].synchronize()
            t = sum(a.elapsed_time(b) for a, b in self.pairs)
        else:
            t = 1e3 * sum(self.pairs)
        if reset:
            self.pairs = []
        return t


class _Null:
    def start(self):
        pass

    def stop(self):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class _Scoped:
    def __init__(self, t):
        self.t = t

    def start(self):
        self.t.start()

    def stop(self):
        self.t.stop()

    def __enter__(self):
        self.t.start()
        return self

    def __exit__(self, *a):
        self.t.stop()
        return False


class Timers:
    def __init__(self, log_level: int = 0, log_option: str = "minmax", cuda: bool = False):
        assert log_option in ("max", "minmax", "all")
        self.log_level, self.log_option, self.cuda = log_level, log_option, cuda
        self.timers: dict[str, _Timer] = {}
        self.last_max_ms: dict[str, float] = {}
        self._null = _Null()

    def __call__(self, name: str, log_level: int = 1):
        """Timer ``name`` (usable as a context manager); a no-op object when its level is above ``timing_log_level``."""
        if log_level > self.log_level:
            return self._null
        t = self.timers.get(name)
        if t is None:
            t = self.timers[name] = _Timer(name, self.cuda)
        return _Scoped(t)

    def log(self, normalizer: float = 1.0, group=None) -> str | None:
        """One string with every timer's time per ``normalizer`` (iterations), reduced over the ranks; None when there
        is nothing to report.  Resets the timers."""
        if not self.timers:
            return None
        names = sorted(self.timers)
        local = torch.tensor([self.timers[n].elapsed_ms() / max(normalizer, 1e-9) for n in names], dtype=torch.float64)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if self.cuda else torch.device("cpu")
            every = [torch.zeros_like(local, device=dev) for _ in range(world)]
            dist.all_gather(every, local.to(dev), group=group)
            table = torch.stack([e.cpu() for e in every])          # [rank, timer]
        else:
            table = local[None]
        lines = []
        if self.log_option == "all":
            lines.append("times across ranks (ms):")
            for j, n in enumerate(names):
                lines.append(f"    {n}: " + ", ".join(f"rank {r}: {table[r, j]:.2f}" for r in range(table.shape[0])))
        elif self.log_option == "minmax":
            lines.append("(min, max) time across ranks (ms):")
            for j, n in enumerate(names):
                lines.append(f"    {n + ' ':.<48s} ({table[:, j].min():.2f}, {table[:, j].max():.2f})")
        else:
            lines.append("max time across ranks (ms):")
            for j, n in enumerate(names):
                lines.append(f"    {n + ' ':.<48s} {table[:, j].max():.2f}")
        # the same numbers for the metric sinks (``log_timers_to_tensorboard``): max over ranks per timer
        self.last_max_ms = {n: float(table[:, j].max()) for j, n in enumerate(names)}
        return "\n".join(lines)
