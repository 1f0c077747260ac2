"""MLPerf-style structured training log: ``:::MLLOG {json}`` lines that the MLPerf compliance tools read.

With ``mlperf_mode`` the trainer emits, on the logging rank: the submission / hyper-parameter header and ``init_start``
while it is built; ``init_stop`` + ``run_start`` + ``epoch_start`` + ``block_start`` before the first step;
``tracked_stats`` (loss, learning rate, samples, throughput) at every logged step; around every evaluation ``block_stop`` /
``eval_start`` / ``eval_accuracy`` (the validation loss) / ``eval_stop`` and the next ``block_start``; and ``run_stop``
with status ``success`` as soon as the validation loss reaches ``mlperf_target_eval_loss`` (training then ends) or
``aborted`` when the run finishes without reaching it.  Training throughput leaves the time spent in evaluation out.

The line format is the one of the ``mlperf_logging.mllog`` package (namespace, ``time_ms``, ``event_type``
POINT_IN_TIME / INTERVAL_START / INTERVAL_END, key, value, metadata with file and line); it is written here directly,
so the package is not needed.  Role of the reference's MLPerf logging patch
(primus/backends/megatron/patches/mlperf_logging_patches.py:78-290: events and their order; ``mlperf_mode`` switch :29-31)."""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Callable, Optional

PREFIX = ":::MLLOG"


class ThroughputClock:
    """Samples per second of training time only: the clock stops while an evaluation runs."""

    def __init__(self, global_batch: int, now: Callable[[], float] = time.time):
        self.gbs, self.now = global_batch, now
        self.start: Optional[float] = None
        self.paused_at: Optional[float] = None
        self.paused = 0.0
        self.samples = 0

    def begin(self):
        if self.start is None:
            self.start = self.now()

    def step(self, n: int = 1):
        self.samples += n * self.gbs

    def pause(self):
        self.paused_at = self.now()

    def resume(self):
        if self.paused_at is not None:
            self.paused += self.now() - self.paused_at
            self.paused_at = None

    def samples_per_s(self, include_eval: bool = False) -> float:
        if self.start is None:
            return 0.0
        t = self.now() - self.start - (0.0 if include_eval else self.paused)
        return self.samples / t if t > 0 else 0.0


class MLPerfLogger:
    def __init__(self, benchmark: str, global_batch: int, target: Optional[float] = None, org: str = "primus_b200",
                 platform: str = "B200", division: str = "closed", enabled: bool = True,
                 sink: Optional[Callable[[str], None]] = None, path: Optional[str] = None,
                 now: Callable[[], float] = time.time):
        self.benchmark, self.gbs, self.target = benchmark, global_batch, target
        self.org, self.platform, self.division = org, platform, division
        self.enabled, self.now = enabled, now
        self._file = open(path, "a") if (path and enabled) else None
        self.sink = sink or (lambda line: print(line, flush=True))
        self.clock = ThroughputClock(global_batch, now)
        self.started = self.stopped = False
        self.converged = False

    # ------------------------------------------------------------------ line format
    def _emit(self, event_type: str, key: str, value=None, metadata: Optional[dict] = None):
        if not self.enabled:
            return
        frame = sys._getframe(2)
        md = {"file": os.path.relpath(frame.f_code.co_filename), "lineno": frame.f_lineno}
        md.update(metadata or {})
        line = f"{PREFIX} " + json.dumps({"namespace": "", "time_ms": int(self.now() * 1000), "event_type": event_type,
                                         "key": key, "value": value, "metadata": md})
        self.sink(line)
        if self._file is not None:
            self._file.write(line + "\n")
            self._file.flush()

    def event(self, key, value=None, metadata=None):
        self._emit("POINT_IN_TIME", key, value, metadata)

    def start(self, key, value=None, metadata=None):
        self._emit("INTERVAL_START", key, value, metadata)

    def end(self, key, value=None, metadata=None):
        self._emit("INTERVAL_END", key, value, metadata)

    # ------------------------------------------------------------------ the run's events, in order
    def log_init(self, seed: int):
        self.start("init_start")
        self.event("submission_benchmark", self.benchmark)
        self.event("submission_org", self.org)
        self.event("submission_division", self.division)
        self.event("submission_platform", self.platform)
        self.event("submission_status", "onprem")
        if self.target is not None:
            self.event("target_accuracy", self.target)
        self.event("seed", seed)

    def log_hyperparams(self, tc, num_microbatches: int, train_samples: int, eval_samples: int):
        self.event("global_batch_size", self.gbs)
        self.event("train_samples", train_samples)
        self.event("eval_samples", eval_samples)
        self.event("gradient_accumulation_steps", num_microbatches)
        self.event("opt_name", "adamw" if tc.optimizer.lower() in ("adam", "adamw") else tc.optimizer.lower())
        self.event("opt_base_learning_rate", tc.lr)
        self.event("opt_learning_rate_warmup_steps", tc.lr_warmup_iters)
        self.event("opt_adamw_beta_1", tc.adam_beta1)
        self.event("opt_adamw_beta_2", tc.adam_beta2)
        self.event("opt_adamw_epsilon", tc.adam_eps)
        self.event("opt_adamw_weight_decay", tc.weight_decay)
        self.event("opt_gradient_clip_norm", tc.clip_grad)
        self.event("max_sequence_length", tc.seq_length)

    def run_start(self):
        if self.started:
            return
        self.started = True
        self.end("init_stop")
        self.start("run_start")
        self.start("epoch_start", metadata={"epoch_num": 0})
        self.start("block_start", metadata={"first_epoch_num": 0, "samples_count": self.clock.samples})
        self.clock.begin()

    def on_step(self, step: int, loss: float, lr: float, steps: int = 1):
        self.clock.step(steps)
        self.event("tracked_stats", {"train_loss": loss, "lr": lr, "throughput": round(self.clock.samples_per_s(), 3)},
                   {"step": step, "samples_count": self.clock.samples})

    def eval_begin(self, step: int):
        self.event("throughput", round(self.clock.samples_per_s(), 3), {"step": step})
        self.end("block_stop", metadata={"first_epoch_num": 0, "samples_count": self.clock.samples})
        self.clock.pause()
        self.start("eval_start", metadata={"epoch_num": 0, "samples_count": self.clock.samples})

    def eval_end(self, step: int, val_loss: float) -> bool:
        """Returns True when the target is reached (the run is over)."""
        self.event("eval_accuracy", val_loss, {"epoch_num": 0, "samples_count": self.clock.samples, "step": step})
        self.end("eval_stop", metadata={"epoch_num": 0, "samples_count": self.clock.samples})
        self.clock.resume()
        self.event("combined_throughput", round(self.clock.samples_per_s(include_eval=True), 3), {"step": step})
        if self.target is not None and val_loss <= self.target:
            self.converged = True
            self.run_stop(True, step)
            return True
        self.start("block_start", metadata={"first_epoch_num": 0, "samples_count": self.clock.samples})
        return False

    def run_stop(self, success: bool, step: int):
        if self.stopped or not self.started:
            return
        self.stopped = True
        self.end("epoch_stop", metadata={"epoch_num": 0})
        self.end("run_stop", metadata={"status": "success" if success else "aborted", "step": step,
                                       "samples_count": self.clock.samples})

    def close(self):
        if self._file is not None:
            self._file.close()
            self._file = None
