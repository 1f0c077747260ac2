"""Projection tool: collective-model math, memory accounting against hand-computed values, plan legality,
monotonic behaviour of the performance model, CLI return codes."""
import subprocess
import sys
import os

import pytest

from primus_b200.core.config.presets import load_preset
from primus_b200.models.config import TransformerConfig
from primus_b200.tools.projection.collective_model import CollectiveModel, Hardware
from primus_b200.tools.projection.memory import ParallelPlan, param_counts, project_memory
from primus_b200.tools.projection.performance import project_performance

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hw(**kw):
    return Hardware.from_yaml({**load_preset("b200", "hardware"), **kw})


def cfg(name):
    return TransformerConfig.from_dict(load_preset(name, "models"))


def test_ring_allreduce_formula_without_nvls():
    h = hw(nvls=False)
    m = CollectiveModel(h)
    S, p = 1 << 30, 8
    bw = h.node_bw_gbs * 1e9 * h.bw_eff
    expect = (h.launch_us + h.ar_overhead_us) * 1e-6 + 2 * ((p - 1) * h.node_lat_us * 1e-6 + S * (p - 1) / p / bw)
    assert abs(m.all_reduce(S, p) - expect) < 1e-9
    assert m.all_reduce(S, 1) == 0 and m.all_to_all(0, 8) == 0
    assert m.reduce_scatter(S, 8) < m.all_reduce(S, 8)


def test_multi_node_is_slower_and_hierarchical():
    m = CollectiveModel(hw())
    S = 256 << 20
    assert m.all_reduce(S, 16) > m.all_reduce(S, 8)
    assert m.all_to_all(S, 64) > m.all_to_all(S, 8)
    assert m.send_recv(S, inter_node=True) > m.send_recv(S, inter_node=False)


def test_param_counts_match_config():
    for name in ("llama3.1_8B", "deepseek_v2_lite", "qwen3_30B_A3B"):
        c = cfg(name)
        pc = param_counts(c)
        total = pc["embedding"] + pc["output"] + sum(l["dense"] + l["expert"] for l in pc["layers"])
        assert abs(total - c.num_parameters()) / c.num_parameters() < 2e-3, name


def test_memory_llama8b_hand_computed():
    c = cfg("llama3.1_8B")
    plan = ParallelPlan(world=8, global_batch=128, seq=8192)
    mem = project_memory(c, plan)
    b = mem["breakdown"]
    n = c.num_parameters()
    assert abs(b["weights_gb"] - n * 2 / 2**30) < 0.1
    assert abs(b["grads_gb"] - n * 4 / 2**30) < 0.1
    assert abs(b["optimizer_gb"] - n * 12 / 8 / 2**30) < 0.1
    one = project_memory(c, ParallelPlan(world=1, global_batch=16, seq=8192))
    assert one["breakdown"]["optimizer_gb"] > 7.9 * b["optimizer_gb"]
    rec = project_memory(c, ParallelPlan(world=8, global_batch=128, seq=8192, recompute_layers=32))
    assert rec["breakdown"]["activations_gb"] < 0.2 * b["activations_gb"]


def test_plan_legality():
    c = cfg("llama3.1_70B")
    assert ParallelPlan(world=8, tp=8, global_batch=64).validate(c) == []
    assert ParallelPlan(world=8, tp=3, global_batch=64).validate(c)
    assert ParallelPlan(world=8, tp=4, pp=2, vpp=3, global_batch=64).validate(c)
    m = cfg("deepseek_v2_lite")
    assert ParallelPlan(world=8, ep=8, global_batch=64, seq=4096).validate(m) == []
    assert ParallelPlan(world=8, ep=5, global_batch=64, seq=4096).validate(m)


def test_performance_model_trends():
    c = cfg("llama3.1_8B")
    h = hw()
    p8 = project_performance(c, ParallelPlan(world=8, global_batch=128), h)
    assert 5000 < p8["tokens_per_s_per_gpu"] < 40000 and 0.2 < p8["mfu"] < 0.95
    p64 = project_performance(c, ParallelPlan(world=8, global_batch=1024), h, target_nodes=8)
    assert p64["world"] == 64 and p64["tokens_per_s_per_gpu"] <= p8["tokens_per_s_per_gpu"] * 1.01
    c70 = cfg("llama3.1_70B")
    base = project_performance(c70, ParallelPlan(world=8, tp=8, global_batch=64), h, comm_overlap=0.0)
    fused = project_performance(c70, ParallelPlan(world=8, tp=8, global_batch=64), h, comm_overlap=0.7)
    assert fused["iteration_ms"] < base["iteration_ms"]
    f1 = project_performance(c70, ParallelPlan(world=8, tp=4, pp=2, global_batch=64), h, schedule="1f1b")
    il = project_performance(c70, ParallelPlan(world=8, tp=4, pp=2, vpp=2, global_batch=64), h, schedule="interleaved")
    assert il["bubble_fraction"] < f1["bubble_fraction"]


@pytest.mark.parametrize("args", [
    ["projection", "memory", "--model", "llama3.1_8B", "--world", "8"],
    ["projection", "performance", "--model", "deepseek_v2_lite", "--world", "8", "--ep", "8", "--global-batch", "64", "--seq", "4096"],
    ["projection", "both", "--config", "examples/configs/llama3.1_70B-BF16-TP4PP2-pretrain.yaml", "--json"],
])
def test_cli_returns_zero(args):
    r = subprocess.run([sys.executable, "-m", "primus_b200.cli.main", *args], capture_output=True, text=True, cwd=ROOT,
                       env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode == 0, r.stderr + r.stdout


def test_tuner_ranks_only_legal_plans_that_fit():
    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig
    from primus_b200.tools.projection.collective_model import Hardware
    from primus_b200.tools.projection.memory import project_memory
    from primus_b200.tools.tuner import search as tuner

    cfg = TransformerConfig.from_dict(load_preset("llama3.1_70B", "models"))
    hw = Hardware.from_yaml(load_preset("b200", "hardware"))
    res = tuner.search(cfg, hw, world=8, global_batch=64, seq=8192, top=5)
    assert res["enumerated"] > res["fit_in_memory"] > 0 and res["best"]
    ts = [c.tokens_per_s_per_gpu for c in res["best"]]
    assert ts == sorted(ts, reverse=True)
    for c in res["best"]:
        assert not c.plan.validate(cfg)
        assert project_memory(cfg, c.plan)["peak_gb"] <= hw.hbm_gb
        assert any(o.startswith("--tensor_model_parallel_size=") for o in c.overrides())
    # an 8B model fits without model parallelism: the pure data-parallel plan is among the candidates that fit
    cfg8 = TransformerConfig.from_dict(load_preset("llama3.1_8B", "models"))
    res8 = tuner.search(cfg8, hw, world=8, global_batch=128, seq=8192, top=1000)
    assert any((c.plan.tp, c.plan.pp, c.plan.cp) == (1, 1, 1) for c in res8["best"])


def test_model_stats_reproduce_known_parameter_counts():
    from primus_b200.tools import model_stats

    rows = {r["model"]: r for r in model_stats.main(["--model", "llama3.1_8B", "qwen3_30B_A3B", "deepseek_v3",
                                                     "mixtral_8x7B_v0.1", "--json"])}
    assert abs(rows["llama3.1_8B"]["params_B"] - 8.03) < 0.02
    assert abs(rows["qwen3_30B_A3B"]["params_B"] - 30.5) < 0.1 and abs(rows["qwen3_30B_A3B"]["active_params_B"] - 3.3) < 0.1
    assert abs(rows["deepseek_v3"]["params_B"] - 671) < 2 and abs(rows["deepseek_v3"]["active_params_B"] - 37.5) < 0.5
    assert abs(rows["mixtral_8x7B_v0.1"]["params_B"] - 46.7) < 0.1


# Measured steps of this package on B200 (device-timed, max over ranks): profiles/bench_llama3.1_8B_*.json.txt,
# profiles/data_parallel_overlap_8gpu_llama3.1_8B.md, profiles/bench_other_configs_8gpu.md
MEASURED_MS = [
    ("llama3.1_8B", dict(world=1, global_batch=16), "1f1b", "mxfp8", 5514.0),
    ("llama3.1_8B", dict(world=8, global_batch=128), "1f1b", "mxfp8", 5642.0),
    ("llama3.1_8B", dict(world=1, global_batch=16), "1f1b", "bf16", 7486.0),
    ("llama3.1_70B", dict(world=8, tp=8, global_batch=4), "1f1b", "mxfp8", 2340.0),
    ("llama3.1_70B", dict(world=8, tp=4, pp=2, vpp=2, global_batch=8), "interleaved", "mxfp8", 3658.0),
]


def test_performance_projection_matches_measured_steps():
    """The kernel table of the performance model is calibrated on measured runs: every projected iteration time must
    stay within 10 % of its measurement (the reference validates its projection against measured runs the same way,
    docs_deprecated/tech_blogs/projection/projection.md:454-456)."""
    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig
    from primus_b200.tools.projection.collective_model import Hardware

    hw = Hardware.from_yaml(load_preset("b200", "hardware"))
    for model, plan_kw, sched, prec, ms in MEASURED_MS:
        cfg = TransformerConfig.from_dict(load_preset(model, "models"))
        got = project_performance(cfg, ParallelPlan(**plan_kw), hw, sched, precision=prec)["iteration_ms"]
        assert abs(got - ms) <= 0.10 * ms, (model, plan_kw, prec, got, ms)
