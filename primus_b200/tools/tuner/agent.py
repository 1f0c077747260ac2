"""Iterative configuration tuning: propose plans, check them, evaluate them, remember everything, repeat.

    python -m primus_b200.tools.tuner.agent --model llama3.1_70B --world 8 --global-batch 64 --seq 8192 \\
        [--rounds 6] [--per-round 8] [--proposer hill|grid|llm] [--evaluate projection|benchmark] \\
        [--history tuning.jsonl] [--config exp.yaml] [--report tuning.md]

One round: the *proposer* suggests parallel plans given the history; every suggestion goes through the *legality*
checks (divisibility rules of the engine, with the reason recorded when one fails) and the *memory* projection (plans
over the HBM size are recorded as such and never run); the survivors are scored by the *evaluator* -- the analytic
performance projection, or a short real training run through the launcher whose log gives tokens/s/GPU -- and appended
to the *history* file, which also makes a search resumable (nothing is evaluated twice).  The report shows the best
plan, the best-so-far curve over the evaluations and the overrides that select the winner.

Proposers: ``grid`` walks the exhaustive enumeration of ``tools/tuner/search.py`` in projected order; ``hill`` starts
from the projection's best plans and then explores the neighbours (one knob changed) of the best measured plans;
``llm`` asks a chat-completion endpoint (``TUNER_LLM_BASE`` / ``TUNER_LLM_MODEL`` / ``TUNER_LLM_KEY``, any
OpenAI-compatible server) for plans as JSON, shows it the model, the cluster and the history, and falls back to ``hill``
when the endpoint is not configured or answers nothing usable -- its suggestions pass the same checks as any other.

Role of the reference's tuning agent (primus/agents/tuning_agent/: ``plan.py`` search space, ``legality.py``,
``evaluator.py`` projection / benchmark oracle, ``history.py``, ``plotting.py``, ``agent.py`` LLM loop)."""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import urllib.request
from typing import Callable, Iterable, Optional

from ..projection.collective_model import Hardware
from ..projection.memory import ParallelPlan, project_memory
from ..projection.performance import project_performance
from . import search as S

KNOBS = ("tp", "pp", "vpp", "ep", "cp", "micro_batch", "recompute_layers", "schedule")


def plan_key(d: dict) -> str:
    return ",".join(f"{k}={d.get(k)}" for k in KNOBS)


def to_plan(d: dict, world: int, global_batch: int, seq: int) -> ParallelPlan:
    tp = int(d.get("tp", 1))
    return ParallelPlan(world=world, tp=tp, pp=int(d.get("pp", 1)), cp=int(d.get("cp", 1)), ep=int(d.get("ep", 1)),
                        vpp=int(d.get("vpp", 1)), micro_batch=int(d.get("micro_batch", 1)), global_batch=global_batch,
                        seq=seq, recompute_layers=int(d.get("recompute_layers", 0)), sequence_parallel=tp > 1,
                        fused_tp=tp > 1)


# ------------------------------------------------------------------------------------------------ checks
def legality(cfg, d: dict, world: int, global_batch: int, seq: int) -> list:
    """Reasons why the engine would reject the plan (empty: legal)."""
    plan = to_plan(d, world, global_batch, seq)
    errs = list(plan.validate(cfg))
    sched = d.get("schedule", "1f1b")
    if plan.pp == 1 and sched != "1f1b":
        errs.append("a pipeline schedule without pipeline stages")
    if plan.vpp > 1 and sched != "interleaved":
        errs.append("virtual stages need the interleaved schedule")
    if plan.vpp == 1 and sched == "interleaved":
        errs.append("the interleaved schedule needs virtual stages")
    if plan.pp > 1 and plan.grad_accum < plan.pp:
        errs.append("fewer micro-batches than pipeline stages")
    if plan.recompute_layers > cfg.num_layers // max(plan.pp * plan.vpp, 1):
        errs.append("more recomputed layers than a stage holds")
    if cfg.num_experts and plan.tp > 1 and not plan.sequence_parallel:
        errs.append("MoE layers under tensor parallelism need sequence parallelism")
    if seq % max(plan.cp * (plan.tp if plan.sequence_parallel else 1), 1):
        errs.append("sequence length not divisible by cp x tp")
    return errs


# ------------------------------------------------------------------------------------------------ evaluators
class ProjectionEvaluator:
    name = "projection"

    def __init__(self, cfg, hw: Hardware, comm_overlap: float = 0.7):
        self.cfg, self.hw, self.comm_overlap = cfg, hw, comm_overlap

    def __call__(self, d: dict, plan: ParallelPlan) -> dict:
        perf = project_performance(self.cfg, plan, self.hw, d.get("schedule", "1f1b"),
                                   comm_overlap=self.comm_overlap if plan.fused_tp else 0.0)
        return {"tokens_per_s_per_gpu": perf["tokens_per_s_per_gpu"], "iteration_ms": perf["iteration_ms"], "mfu": perf["mfu"]}


class BenchmarkEvaluator:
    """A short real run of the experiment config with the plan's overrides; the score is what the training log reports."""
    name = "benchmark"

    def __init__(self, config: str, launcher: str, log_dir: str, iters: int = 8, skip: int = 3, timeout: float = 1800.0):
        self.config, self.launcher, self.log_dir, self.iters, self.skip, self.timeout = config, launcher, log_dir, iters, skip, timeout
        self.runs = 0

    def __call__(self, d: dict, plan: ParallelPlan) -> dict:
        from ..ops.auto_benchmark import run_config

        self.runs += 1
        cand = S.Candidate(plan, d.get("schedule", "1f1b"), 0.0, 0.0, 0.0, 0.0, 0.0)
        ov = [o.lstrip("-") for o in cand.overrides()] + [f"train_iters={self.iters}", "mock_data=true"]
        os.makedirs(self.log_dir, exist_ok=True)
        rec = run_config(self.config, self.launcher, os.path.join(self.log_dir, f"cand{self.runs:03d}"), ov, self.timeout, False)
        if rec.get("status") != "ok":
            raise RuntimeError(f"run {rec.get('status')} (see {self.log_dir}/cand{self.runs:03d})")
        return {"tokens_per_s_per_gpu": rec["tokens_s_gpu"], "iteration_ms": rec["ms_per_iter"], "max_mem_gib": rec["max_mem_gib"]}


# ------------------------------------------------------------------------------------------------ history
class History:
    def __init__(self, path: Optional[str] = None):
        self.path, self.records = path, []
        if path and os.path.exists(path):
            with open(path) as f:
                self.records = [json.loads(line) for line in f if line.strip()]

    def seen(self) -> set:
        return {plan_key(r["plan"]) for r in self.records}

    def add(self, rec: dict) -> None:
        self.records.append(rec)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")

    def evaluated(self) -> list:
        return [r for r in self.records if r["status"] == "evaluated"]

    def best(self, n: int = 1) -> list:
        return sorted(self.evaluated(), key=lambda r: -r["tokens_per_s_per_gpu"])[:n]

    def best_so_far(self) -> list:
        out, best = [], 0.0
        for r in self.evaluated():
            best = max(best, r["tokens_per_s_per_gpu"])
            out.append(best)
        return out


# ------------------------------------------------------------------------------------------------ proposers
def neighbours(d: dict, cfg, world: int) -> Iterable[dict]:
    """Plans one knob away: a factor of two in a parallel degree or the micro-batch, recompute on / off, the schedule."""
    for k in ("tp", "pp", "cp", "ep", "micro_batch", "vpp"):
        for f in (0.5, 2):
            v = int(d.get(k, 1) * f)
            if v >= 1 and v != d.get(k, 1):
                n = dict(d, **{k: v})
                if k == "pp" and v == 1:
                    n.update(vpp=1, schedule="1f1b")
                if k == "vpp":
                    n["schedule"] = "interleaved" if v > 1 else "1f1b"
                yield n
    per_stage = cfg.num_layers // max(d.get("pp", 1) * d.get("vpp", 1), 1)
    yield dict(d, recompute_layers=0 if d.get("recompute_layers") else per_stage)
    if d.get("pp", 1) > 1 and d.get("vpp", 1) == 1:
        yield dict(d, schedule="zerobubble" if d.get("schedule") == "1f1b" else "1f1b")


class GridProposer:
    name = "grid"

    def __init__(self, cfg, hw, world, global_batch, seq):
        res = S.search(cfg, hw, world, global_batch, seq, top=10 ** 6)
        self.queue = [c.as_dict() for c in res["best"]]

    def propose(self, history: History, n: int) -> list:
        seen = history.seen()
        out = [d for d in self.queue if plan_key(d) not in seen][:n]
        return out


class HillProposer(GridProposer):
    name = "hill"

    def __init__(self, cfg, hw, world, global_batch, seq):
        super().__init__(cfg, hw, world, global_batch, seq)
        self.cfg, self.world = cfg, world

    def propose(self, history: History, n: int) -> list:
        seen = history.seen()
        out, keys = [], set()
        for r in history.best(3):
            for nb in neighbours(r["plan"], self.cfg, self.world):
                k = plan_key(nb)
                if k not in seen and k not in keys:
                    keys.add(k)
                    out.append({x: nb.get(x, 1 if x != "schedule" else "1f1b") for x in KNOBS})
        for d in self.queue:               # fill up (and start) with the projection's favourites
            if len(out) >= n:
                break
            k = plan_key(d)
            if k not in seen and k not in keys:
                keys.add(k)
                out.append({x: d[x] for x in KNOBS})
        return out[:n]


class LLMProposer(HillProposer):
    """Chat-completion endpoint as proposer.  ``transport(payload) -> text`` can be injected (tests, other clients)."""
    name = "llm"

    def __init__(self, cfg, hw, world, global_batch, seq, transport: Optional[Callable[[dict], str]] = None):
        super().__init__(cfg, hw, world, global_batch, seq)
        self.hw, self.global_batch, self.seq = hw, global_batch, seq
        self.transport = transport or self._http
        self.fallbacks = 0

    @staticmethod
    def _http(payload: dict) -> str:
        base = os.environ.get("TUNER_LLM_BASE")
        if not base:
            raise RuntimeError("TUNER_LLM_BASE is not set")
        req = urllib.request.Request(base.rstrip("/") + "/chat/completions", data=json.dumps(payload).encode(),
                                     headers={"Content-Type": "application/json",
                                              "Authorization": "Bearer " + os.environ.get("TUNER_LLM_KEY", "none")})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.load(r)["choices"][0]["message"]["content"]

    def prompt(self, history: History, n: int) -> str:
        c = self.cfg
        rows = [dict(r["plan"], status=r["status"], tokens_per_s_per_gpu=round(r.get("tokens_per_s_per_gpu", 0), 1),
                     reason=r.get("reason", "")) for r in history.records[-40:]]
        return (f"Model: {c.num_layers} layers, hidden {c.hidden_size}, {c.num_attention_heads} heads, "
                f"{c.num_experts or 0} experts. Cluster: {self.world} x {self.hw.name}, {self.hw.hbm_gb:.0f} GB each, "
                f"{self.hw.gpus_per_node} per node. Global batch {self.global_batch}, sequence {self.seq}.\n"
                f"History (newest last): {json.dumps(rows)}\n"
                f"Propose {n} new plans likely to beat the best tokens_per_s_per_gpu. Answer with a JSON list of objects "
                f"with the keys {list(KNOBS)} (schedule: 1f1b | interleaved | zerobubble) and nothing else.")

    def propose(self, history: History, n: int) -> list:
        try:
            text = self.transport({"model": os.environ.get("TUNER_LLM_MODEL", "default"), "temperature": 0.3,
                                   "messages": [{"role": "system", "content": "You tune distributed training plans."},
                                                {"role": "user", "content": self.prompt(history, n)}]})
            plans = json.loads(text[text.index("["): text.rindex("]") + 1])
            seen = history.seen()
            out = [{k: p.get(k, "1f1b" if k == "schedule" else 1) for k in KNOBS} for p in plans if isinstance(p, dict)]
            out = [p for p in out if plan_key(p) not in seen]
            if out:
                return out[:n]
        except Exception:  # noqa: BLE001  (no endpoint, a timeout, prose instead of JSON: the search goes on without it)
            pass
        self.fallbacks += 1
        return super().propose(history, n)


# ------------------------------------------------------------------------------------------------ the loop
def tune(cfg, hw: Hardware, world: int, global_batch: int, seq: int, proposer, evaluator, history: History,
         rounds: int = 6, per_round: int = 8, hbm_gb: Optional[float] = None, log=print) -> History:
    hbm = hbm_gb or hw.hbm_gb
    for rnd in range(rounds):
        batch = proposer.propose(history, per_round)
        if not batch:
            log(f"round {rnd}: nothing left to propose")
            break
        for d in batch:
            if plan_key(d) in history.seen():
                continue
            rec = {"round": rnd, "plan": {k: d.get(k) for k in KNOBS}, "proposer": proposer.name}
            errs = legality(cfg, d, world, global_batch, seq)
            if errs:
                history.add(dict(rec, status="illegal", reason="; ".join(errs)))
                continue
            plan = to_plan(d, world, global_batch, seq)
            peak = project_memory(cfg, plan)["peak_gb"]
            if peak > hbm:
                history.add(dict(rec, status="out_of_memory", peak_gb=round(peak, 1), reason=f"{peak:.0f} GB projected, {hbm:.0f} GB available"))
                continue
            try:
                score = evaluator(d, plan)
            except Exception as e:  # noqa: BLE001  (a schedule that cannot be built, a run that failed)
                history.add(dict(rec, status="failed", peak_gb=round(peak, 1), reason=f"{type(e).__name__}: {e}"))
                continue
            history.add(dict(rec, status="evaluated", peak_gb=round(peak, 1), evaluator=evaluator.name, **score))
        best = history.best(1)
        if best:
            log(f"round {rnd}: {len(batch)} proposed, best so far {best[0]['tokens_per_s_per_gpu']:.0f} tokens/s/GPU "
                f"with {plan_key(best[0]['plan'])}")
    return history


def text_curve(values: list, width: int = 60, height: int = 8) -> str:
    """Best-so-far curve as a small character plot."""
    if not values:
        return "(nothing evaluated)"
    lo, hi = min(values), max(values)
    cols = [values[min(len(values) - 1, int(i * len(values) / width))] for i in range(min(width, len(values)))]
    rows = []
    for h in range(height, 0, -1):
        cut = lo + (hi - lo) * (h - 0.5) / height
        rows.append(f"{cut:10.0f} |" + "".join("#" if v >= cut else " " for v in cols))
    return "\n".join(rows + [" " * 11 + "+" + "-" * len(cols), " " * 12 + f"evaluations 1..{len(values)}"])


def report(history: History, world: int, global_batch: int, seq: int) -> str:
    counts = {}
    for r in history.records:
        counts[r["status"]] = counts.get(r["status"], 0) + 1
    lines = [f"plans: {len(history.records)} ({', '.join(f'{v} {k}' for k, v in sorted(counts.items()))})", ""]
    best = history.best(5)
    if best:
        lines += ["| " + " | ".join(list(KNOBS) + ["peak GB", "tokens/s/GPU", "evaluator"]) + " |",
                  "|" + "---|" * (len(KNOBS) + 3)]
        for r in best:
            lines.append("| " + " | ".join(str(r["plan"][k]) for k in KNOBS) +
                         f" | {r.get('peak_gb', '')} | {r['tokens_per_s_per_gpu']:.0f} | {r.get('evaluator', '')} |")
        top = best[0]
        cand = S.Candidate(to_plan(top["plan"], world, global_batch, seq), top["plan"]["schedule"], 0, 0, 0, 0, 0)
        lines += ["", "best so far over the evaluations:", "```", text_curve(history.best_so_far()), "```", "",
                  "overrides of the best plan: `" + " ".join(cand.overrides()) + "`"]
    return "\n".join(lines)


def main(argv=None) -> int:
    from ...core.config.presets import load_preset
    from ...models.config import TransformerConfig

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama3.1_70B")
    ap.add_argument("--hardware", default="b200")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--rounds", type=int, default=6)
    ap.add_argument("--per-round", type=int, default=8)
    ap.add_argument("--proposer", default="hill", choices=["grid", "hill", "llm"])
    ap.add_argument("--evaluate", default="projection", choices=["projection", "benchmark"])
    ap.add_argument("--config", default=None, help="experiment YAML for --evaluate benchmark")
    ap.add_argument("--launcher", default=os.path.join(os.path.dirname(__file__), "..", "..", "..", "primus-cli"))
    ap.add_argument("--history", default=None)
    ap.add_argument("--report", default=None)
    a = ap.parse_args(argv)
    cfg = TransformerConfig.from_dict(load_preset(a.model, "models"))
    hw = Hardware.from_yaml(load_preset(a.hardware, "hardware"))
    proposer = {"grid": GridProposer, "hill": HillProposer, "llm": LLMProposer}[a.proposer](cfg, hw, a.world, a.global_batch, a.seq)
    if a.evaluate == "benchmark":
        if not a.config:
            ap.error("--evaluate benchmark needs --config")
        evaluator = BenchmarkEvaluator(a.config, os.path.normpath(a.launcher), "output/tuning_agent")
    else:
        evaluator = ProjectionEvaluator(cfg, hw)
    hist = tune(cfg, hw, a.world, a.global_batch, a.seq, proposer, evaluator, History(a.history), a.rounds, a.per_round)
    text = report(hist, a.world, a.global_batch, a.seq)
    print(text)
    if a.report:
        with open(a.report, "w") as f:
            f.write(text + "\n")
    return 0 if hist.best(1) else 1


if __name__ == "__main__":
    sys.exit(main())
