"""Profiling hooks and metric sinks of the training loop.

* :class:`StepProfiler` — ``torch.profiler`` with the schedule the reference installs (skip ``profile_step_start - 1``
  steps, one warm-up step, ``profile_step_end - profile_step_start`` active steps, once), restricted to
  ``profile_ranks``; traces are written as Chrome / TensorBoard-plugin JSON with the worker name
  ``primus-b200-exp[<exp>]-rank[<r>]`` (primus/backends/megatron/patches/torch_profiler_patches.py:20-105;
  keys ``profile, use_pytorch_profiler, profile_ranks, profile_step_start/end, record_memory_history,
  memory_snapshot_path`` of trainer_base.yaml:302-312).  ``record_memory_history`` dumps the CUDA caching-allocator
  history when the profiled window closes.  NVTX ranges around the phases of a step are pushed when ``nvtx_ranges``.
* :class:`MetricsWriter` — per-iteration scalars to every enabled sink: a JSON-lines file (always, when a directory is
  configured), TensorBoard, Weights & Biases and MLflow when the packages are importable (they are optional; a
  missing package disables that sink with one log line, as the reference's writers do:
  primus/backends/megatron/training/global_vars.py:71-137).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Optional

import torch


class StepProfiler:
    def __init__(self, enabled: bool, rank: int, start: int = 3, end: int = 4, ranks=None, out_dir: Optional[str] = None,
                 exp_name: str = "exp", with_cpu: bool = True, record_shapes: bool = True, with_stack: bool = False,
                 use_gzip: bool = False, record_memory_history: bool = False, memory_snapshot_path: Optional[str] = None, log=print):
        self.rank, self.log = rank, log
        self.enabled = bool(enabled) and (ranks is None or rank in ranks)
        self.out_dir = out_dir or os.path.join(os.getcwd(), "profiler")
        self.memory_history = record_memory_history and torch.cuda.is_available()
        self.memory_snapshot_path = memory_snapshot_path or os.path.join(self.out_dir, f"memory_rank{rank}.pickle")
        self.prof = None
        self.end = end
        self.steps = 0
        if not self.enabled:
            return
        os.makedirs(self.out_dir, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else []
        if with_cpu or not acts:
            acts.append(torch.profiler.ProfilerActivity.CPU)
        worker = f"primus-b200-exp[{exp_name}]-rank[{rank}]"

        def handler(p):
            path = os.path.join(self.out_dir, f"{worker}.{int(time.time())}.pt.trace.json" + (".gz" if use_gzip else ""))
            p.export_chrome_trace(path)
            self.log(f"[profiler] trace written to {path}")

        self.prof = torch.profiler.profile(
            activities=acts, record_shapes=record_shapes, with_stack=with_stack, on_trace_ready=handler,
            schedule=torch.profiler.schedule(wait=max(start - 1, 0), warmup=1, active=max(end - start, 1), repeat=1))
        if self.memory_history:
            torch.cuda.memory._record_memory_history(max_entries=100000)
        self.prof.__enter__()

    def step(self):
        if self.prof is None:
            return
        self.steps += 1
        self.prof.step()
        if self.steps == self.end + 1:
            self.close()

    def close(self):
        if self.prof is None:
            return
        self.prof.__exit__(None, None, None)
        self.prof = None
        if self.memory_history:
            try:
                torch.cuda.memory._dump_snapshot(self.memory_snapshot_path)
                torch.cuda.memory._record_memory_history(enabled=None)
                self.log(f"[profiler] memory snapshot written to {self.memory_snapshot_path}")
            except Exception as e:  # noqa: BLE001
                self.log(f"[profiler] memory snapshot failed: {e}")


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class MetricsWriter:
    def __init__(self, rank: int, is_writer_rank: bool, log_dir: Optional[str] = None, tensorboard: bool = False,
                 wandb_project: Optional[str] = None, mlflow_experiment: Optional[str] = None, run_name: str = "run",
                 config: Optional[dict] = None, log=print, wandb_options: Optional[dict] = None):
        """``wandb_options``: extra keyword arguments of ``wandb.init`` (``name``: wandb_exp_name, ``entity``, ``dir``)."""
        self.sinks = []
        self.jsonl = None
        if not is_writer_rank:
            return
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)
            self.jsonl = open(os.path.join(log_dir, "metrics.jsonl"), "a")
        if tensorboard and log_dir:
            try:
                from torch.utils.tensorboard import SummaryWriter

                tb = SummaryWriter(log_dir=log_dir)
                self.sinks.append(("tensorboard", lambda it, m, tb=tb: [tb.add_scalar(k, v, it) for k, v in m.items()],
                                   tb.close))
            except Exception as e:  # noqa: BLE001
                log(f"[metrics] tensorboard sink disabled: {e}")
        if wandb_project:
            try:
                import wandb

                kw = dict(name=run_name, config=config or {})
                kw.update({k: v for k, v in (wandb_options or {}).items() if v})
                run = wandb.init(project=wandb_project, **kw)
                self.sinks.append(("wandb", lambda it, m: wandb.log(m, step=it), run.finish))
            except Exception as e:  # noqa: BLE001
                log(f"[metrics] wandb sink disabled: {e}")
        if mlflow_experiment:
            try:
                import mlflow

                mlflow.set_experiment(mlflow_experiment)
                mlflow.start_run(run_name=run_name)
                self.sinks.append(("mlflow", lambda it, m: mlflow.log_metrics(m, step=it), mlflow.end_run))
            except Exception as e:  # noqa: BLE001
                log(f"[metrics] mlflow sink disabled: {e}")

    def write(self, iteration: int, metrics: dict):
        scalars = {k: float(v) for k, v in metrics.items() if isinstance(v, (int, float)) and k != "iteration"}
        if self.jsonl is not None:
            self.jsonl.write(json.dumps({"iteration": iteration, **scalars}) + "\n")
            self.jsonl.flush()
        for _, fn, _ in self.sinks:
            fn(iteration, scalars)

    def log_artifacts(self, paths, artifact_dir: Optional[str] = None, subdir: str = "artifacts", log=print) -> list:
        """Hand files (profiler traces, trace reports, log files) to the sinks that keep artifacts: they are copied under
        ``<artifact_dir>/<subdir>/`` (always, on the writer rank) and logged to MLflow / W&B when those sinks are
        active.  The upload switches of the reference (``mlflow_upload_traces``, ``mlflow_upload_logs``,
        ``mlflow_upload_tracelens_report``) map onto this call."""
        import shutil

        kept = []
        if artifact_dir:
            dst = os.path.join(artifact_dir, subdir)
            os.makedirs(dst, exist_ok=True)
            for p_ in paths:
                if os.path.isfile(p_):
                    kept.append(shutil.copy2(p_, dst))
        for name, _, _ in self.sinks:
            try:
                if name == "mlflow":
                    import mlflow

                    for p_ in paths:
                        mlflow.log_artifact(p_, artifact_path=subdir)
                elif name == "wandb":
                    import wandb

                    for p_ in paths:
                        wandb.save(p_)
            except Exception as e:  # noqa: BLE001
                log(f"[metrics] {name}: artifact upload failed: {e}")
        return kept

    def close(self):
        if self.jsonl is not None:
            self.jsonl.close()
            self.jsonl = None
        for _, _, closer in self.sinks:
            try:
                closer()
            except Exception:  # noqa: BLE001
                pass
        self.sinks = []
