"""Small tools: the table writer and the SFT data inspector."""
import gzip
import json

import torch

from primus_b200.tools import report


def test_table_writer_formats_and_append(tmp_path, capsys):
    hdr, rows = ["shape", "tflops"], [["8192x4096", 1400.5], ["4096x4096", 1320.0]]
    md = tmp_path / "r.md"
    report.write_table(str(md), hdr, rows, preamble="# GEMM")
    report.write_table(str(md), hdr, [["2048x2048", 900]], append=True)
    text = md.read_text()
    assert text.startswith("# GEMM\n\n| shape | tflops |\n|---|---|\n") and text.count("| shape |") == 1
    assert text.rstrip().endswith("| 2048x2048 | 900 |")
    csvf = tmp_path / "r.csv.gz"
    report.write_table(str(csvf), hdr, rows)
    report.write_table(str(csvf), hdr, rows[:1], append=True)
    lines = gzip.open(csvf, "rt").read().strip().splitlines()
    assert lines[0] == "shape,tflops" and len(lines) == 4
    jl = tmp_path / "r.jsonl"
    report.write_records(str(jl), [{"a": 1, "b": 2}, {"a": 3, "c": 4}])
    recs = [json.loads(l) for l in jl.read_text().splitlines()]
    assert recs == [{"a": 1, "b": 2, "c": ""}, {"a": 3, "b": "", "c": 4}]
    report.write_table("-", hdr, rows)
    assert "| 8192x4096 | 1400.5 |" in capsys.readouterr().out
    assert report.table_format("x.tsv.gz") == "tsv" and report.table_format("noext") == "md"


def test_sft_inspector_reports_mask_and_boundaries(tmp_path, capsys):
    from primus_b200.engine import sft as S
    from primus_b200.tools.diag import inspect_sft_data as I

    recs = [{"instruction": "add", "input": "1 2", "output": "3"}, {"instruction": "say hi", "input": "", "output": "hi"}]
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in recs))
    tok = S.ByteTokenizer()
    ds = S.PackedSFTDataset(S.SFTDataset.from_jsonl(str(data), tok, 512, "alpaca"))
    d = I.describe(ds[0], tok)
    assert d["tokens"] == 512 and 0 < d["supervised"] < 20 and d["num_switches"] == 4      # two answer spans
    assert d["targets_across_boundaries"] == [] and len(d["boundaries"]) >= 3
    bad = dict(ds[0])                      # labels shifted over the whole pack, everything supervised
    bad["labels"] = torch.roll(bad["tokens"], -1)
    bad["loss_mask"] = torch.ones(512)
    assert I.describe(bad, tok)["targets_across_boundaries"]
    assert I.main(["--jsonl", str(data), "--seq-length", "512", "--pack", "--num-samples", "1"]) == 0
    assert "supervised_share" in capsys.readouterr().out


def test_trace_report_categories_overlap_and_files(tmp_path):
    from primus_b200.tools import trace_report as T

    ev = lambda name, ts, dur, cat="kernel", stream=7: {"ph": "X", "cat": cat, "name": name, "ts": ts, "dur": dur,
                                                         "args": {"stream": stream}}
    events = [ev("gemm_mxfp8_kernel<256,0,0,0>", 0, 100), ev("gemm_mxfp8_kernel<256,0,0,0>", 100, 100),
              ev("flash_attn_fwd_kernel<128,128,false>", 200, 50), ev("ncclDevKernel_AllGather", 150, 100, stream=9),
              ev("rmsnorm_fwd_kernel<2>", 300, 10), ev("Memcpy DtoD", 310, 5, cat="gpu_memcpy"),
              {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 500},      # host events are ignored
              ev("quant_mxfp8_kernel", 400, 20)]
    trace = tmp_path / "primus-b200-exp[x]-rank[3].123.pt.trace.json"
    trace.write_text(json.dumps({"traceEvents": events}))
    assert T.categorize("dp_reduce_scatter_kernel") == "collectives" and T.categorize("weird") == "other"
    res = T.analyse(T.load_trace(str(trace)))
    cats = {c["category"]: c for c in res["categories"]}
    assert cats["gemm"]["launches"] == 2 and cats["gemm"]["total_ms"] == 0.2
    assert cats["attention"]["total_ms"] == 0.05 and cats["collectives"]["launches"] == 1
    s = res["summary"]
    assert s["window_us"] == 420 and s["gpu_busy_us"] == 285 and s["comm_hidden_share"] == 1.0
    assert res["top_kernels"][0]["kernel"].startswith("gemm_mxfp8_kernel")
    files = T.write_report(T.find_traces(str(tmp_path)), str(tmp_path / "out"))
    assert [f.split("/")[-1] for f in files] == ["trace_report_rank3.md", "summary.md"]
    text = (tmp_path / "out" / "trace_report_rank3.md").read_text()
    assert "## Top kernels" in text and "| gemm |" in text and "| kernel | category |" in text
    assert T.write_report([str(trace)], str(tmp_path / "o2"), ranks=[0]) == []
    assert T.main([str(tmp_path), "--format", "csv", "--output", str(tmp_path / "o3")]) == 0
    assert (tmp_path / "o3" / "summary.csv").exists()


def test_trainer_writes_a_trace_report_after_the_profiled_window(tmp_path):
    """profile + generate_tracelens_report on CPU: the trace exists, the report step runs and never fails the run (CPU
    traces hold no GPU kernels, so the report is empty but present), and artifacts are copied."""
    import os

    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    out = tmp_path / "tb"
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=4, layers=2, extra_tc=dict(
        profile=True, profile_step_start=2, profile_step_end=3, tensorboard_dir=str(out), generate_tracelens_report=True,
        mlflow_upload_traces=True))
    logs = []
    tr = Trainer(mc, tc, device="cpu", log_fn=logs.append)
    tr.train()
    ps.destroy_model_parallel()
    traces = [f for f in os.listdir(out / "profiler") if f.endswith(".pt.trace.json")]
    assert traces and any("[profiler] trace report" in l for l in logs), logs[-5:]
    assert os.path.isdir(out / "profiler" / "trace_report")
    assert os.listdir(out / "artifacts") == traces


def test_node_bisection_finds_bad_nodes_hangs_and_scale_only_failures(tmp_path):
    from primus_b200.tools.ops import bisect_nodes as B

    assert B.expand_nodelist("a,n[01-03,7]x,b") == ["a", "n01x", "n02x", "n03x", "n7x", "b"]
    nodes = [f"n{i:02d}" for i in range(16)]
    # a real command: fails when a bad node is on the list
    (tmp_path / "check.py").write_text("import sys\nsys.exit(int(bool(set(sys.argv[1].split(',')) & set(['n05', 'n12']))))\n")
    cmd = f"python {tmp_path / 'check.py'} {{nodes}}"
    res = B.bisect(nodes, cmd, timeout=60, jobs=2)
    assert sorted(res.suspects) == ["n05", "n12"] and not res.scale_only
    assert res.trials[0].status == "FAIL" and len(res.trials[0].nodes) == 16
    # a hang is a failure of its own kind, and its process group is gone afterwards
    res = B.bisect(["a", "b"], "python -c \"import time, sys; time.sleep(30 if 'b' in '{nodes}'.split(',') else 0)\"",
                   timeout=1.5, jobs=2)
    assert res.suspects == ["b"] and {t.status for t in res.trials} == {"HANG", "PASS"}
    # fails only with all nodes together
    def runner(template, ns, timeout):
        return B.Trial(list(ns), "FAIL" if len(ns) == 8 else "PASS", 0.0)
    res = B.bisect(nodes[:8], "x", runner=runner)
    assert not res.suspects and res.scale_only == [nodes[:8]]
    out = tmp_path / "bisect.json"
    assert B.main(["--nodes", "a,b", "--command", "true", "--output", str(out)]) == 0
    assert json.loads(out.read_text())["suspects"] == []


def test_auto_benchmark_log_metrics_and_periodic_report(tmp_path):
    from primus_b200.tools.ops import auto_benchmark as A
    from primus_b200.tools.ops import periodic_report as P

    def line(i, ms, tf, tps, loss, mem):
        return (f"[rank0]  iteration {i:8d}/{5:8d} | elapsed time per iteration (ms): {ms:.1f} | throughput per GPU "
                f"(TFLOP/s/GPU): {tf:.1f} | tokens/s/GPU: {tps:.1f} (avg {tps:.1f}) | learning rate: 3.000000E-04 | "
                f"global batch size:   128 | lm loss: {loss:.6E} | grad norm: 1.000 | max mem (GiB): {mem:.2f} |\n")

    text = "".join(line(i, 900.0 if i < 3 else 500.0, 700.0, 20000.0 + i, 10.0 - i, 100.0 + i) for i in range(1, 6))
    rec = A.parse_log(text + "Training completed.\n", skip=2)
    assert rec == dict(iterations=5, completed=True, ms_per_iter=500.0, tflops_gpu=700.0, tokens_s_gpu=20004.0,
                       last_loss=5.0, max_mem_gib=105.0)
    assert A.parse_log("nothing here")["iterations"] == 0
    (tmp_path / "a.log").write_text(text + "Training completed.\n")
    out = tmp_path / "t.jsonl"
    assert A.main(["--parse-logs", str(tmp_path / "a.log"), "--output", str(out)]) == 0
    assert json.loads(out.read_text().splitlines()[0])["tokens_s_gpu"] == 20004.0
    assert A.main(["--configs", "examples/configs/llama_tiny-pretrain.yaml", "--dry-run", "--set", "train_iters=3",
                   "--log-dir", str(tmp_path / "logs")]) == 0
    hist = tmp_path / "hist"
    hist.mkdir()
    (hist / "2026-01-01.jsonl").write_text("\n".join(json.dumps(r) for r in [
        dict(config="a", tokens_s_gpu=100.0, status="ok"), dict(config="b", tokens_s_gpu=100.0, status="ok"),
        dict(config="c", tokens_s_gpu=100.0, status="ok"), dict(config="old", tokens_s_gpu=1.0, status="ok")]))
    (hist / "2026-01-02.jsonl").write_text("\n".join(json.dumps(r) for r in [
        dict(config="a", tokens_s_gpu=101.0, status="ok"), dict(config="b", tokens_s_gpu=90.0, status="ok"),
        dict(config="c", tokens_s_gpu="", status="failed"), dict(config="fresh", tokens_s_gpu=5.0, status="ok")]))
    rows = {r["config"]: r["verdict"] for r in P.compare(P.load_table(str(hist / "2026-01-01.jsonl")),
                                                          P.load_table(str(hist / "2026-01-02.jsonl")), "tokens_s_gpu", 0.03)}
    assert rows == dict(a="same", b="regression", c="failed", fresh="new", old="gone")
    assert P.main(["--history", str(hist), "--output", str(tmp_path / "r.md")]) == 1
    assert "regression" in (tmp_path / "r.md").read_text()


def test_merge_traces_keeps_ranks_apart(tmp_path):
    import gzip

    from primus_b200.tools.ops import merge_traces as M

    for r in (0, 1):
        doc = {"traceEvents": [{"ph": "M", "name": "process_name", "pid": 7, "args": {"name": "python"}},
                               {"ph": "X", "name": f"kernel{r}", "pid": 7, "tid": 1, "ts": 10 * r, "dur": 5}]}
        path = tmp_path / f"rank[{r}].123.pt.trace.json"
        if r:
            with gzip.open(str(path) + ".gz", "wt") as f:
                json.dump(doc, f)
        else:
            path.write_text(json.dumps(doc))
    out = tmp_path / "merged.json.gz"
    assert M.main([str(tmp_path), "--output", str(out)]) == 0
    with gzip.open(out, "rt") as f:
        ev = json.load(f)["traceEvents"]
    assert sorted({e["pid"] for e in ev}) == [7, 100007]
    assert {e["args"]["name"] for e in ev if e["ph"] == "M"} == {"rank 0 python", "rank 1 python"}


def test_tuning_agent_loop_history_legality_and_llm_fallback(tmp_path):
    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig
    from primus_b200.tools.projection.collective_model import Hardware
    from primus_b200.tools.tuner import agent as A

    cfg = TransformerConfig.from_dict(load_preset("llama3.1_70B", "models"))
    hw = Hardware.from_yaml(load_preset("b200", "hardware"))
    world, gbs, seq = 8, 64, 8192
    assert A.legality(cfg, dict(tp=8, pp=1, vpp=1, ep=1, cp=1, micro_batch=1, schedule="1f1b"), world, gbs, seq) == []
    bad = A.legality(cfg, dict(tp=3, pp=1, vpp=2, ep=1, cp=1, micro_batch=1, schedule="zerobubble"), world, gbs, seq)
    assert any("divisible" in e for e in bad) and any("virtual stages" in e for e in bad)
    hist_path = tmp_path / "h.jsonl"
    hist = A.tune(cfg, hw, world, gbs, seq, A.HillProposer(cfg, hw, world, gbs, seq), A.ProjectionEvaluator(cfg, hw),
                  A.History(str(hist_path)), rounds=3, per_round=6, log=lambda m: None)
    assert len(hist.evaluated()) >= 6 and hist.best(1)[0]["tokens_per_s_per_gpu"] > 0
    curve = hist.best_so_far()
    assert all(b >= a for a, b in zip(curve, curve[1:]))
    keys = [A.plan_key(r["plan"]) for r in hist.records]
    assert len(keys) == len(set(keys))                                   # nothing evaluated twice
    # resumed from the file: the second search continues with new plans only
    again = A.tune(cfg, hw, world, gbs, seq, A.HillProposer(cfg, hw, world, gbs, seq), A.ProjectionEvaluator(cfg, hw),
                   A.History(str(hist_path)), rounds=1, per_round=4, log=lambda m: None)
    keys2 = [A.plan_key(r["plan"]) for r in again.records]
    assert keys2[:len(keys)] == keys and len(set(keys2)) == len(keys2) > len(keys)
    # a 70B model on one GPU: every plan is stopped by the memory projection, none is run
    one = A.tune(cfg, hw, 1, 8, seq, A.GridProposer.__new__(A.GridProposer), A.ProjectionEvaluator(cfg, hw), A.History(),
                 rounds=0, log=lambda m: None)
    assert not one.records
    hist1 = A.History()
    p = A.HillProposer.__new__(A.HillProposer)
    p.cfg, p.world, p.queue = cfg, 1, [dict(tp=1, pp=1, vpp=1, ep=1, cp=1, micro_batch=1, recompute_layers=0, schedule="1f1b")]
    A.tune(cfg, hw, 1, 8, seq, p, A.ProjectionEvaluator(cfg, hw), hist1, rounds=1, per_round=1, log=lambda m: None)
    assert hist1.records[0]["status"] == "out_of_memory"
    # the language-model proposer: usable JSON is taken (after the same checks), anything else falls back to hill climbing
    answers = iter(['Sure! [{"tp": 8, "pp": 1, "vpp": 1, "ep": 1, "cp": 1, "micro_batch": 2, "recompute_layers": 0, '
                    '"schedule": "1f1b"}, {"tp": 5, "pp": 1, "micro_batch": 1}]', "I cannot help with that."])
    llm = A.LLMProposer(cfg, hw, world, gbs, seq, transport=lambda payload: next(answers))
    h2 = A.tune(cfg, hw, world, gbs, seq, llm, A.ProjectionEvaluator(cfg, hw), A.History(), rounds=2, per_round=3,
                log=lambda m: None)
    by_status = {}
    for r in h2.records:
        by_status.setdefault(r["status"], []).append(r)
    assert by_status["illegal"][0]["plan"]["tp"] == 5 and llm.fallbacks == 1 and len(h2.evaluated()) >= 2
    assert "tokens_per_s_per_gpu" in llm.prompt(h2, 3)
    text = A.report(hist, world, gbs, seq)
    assert "overrides of the best plan" in text and "#" in text
    assert A.main(["--model", "llama3.1_8B", "--world", "8", "--global-batch", "128", "--rounds", "1", "--per-round", "3",
                   "--report", str(tmp_path / "r.md")]) == 0


def test_config_reference_is_current():
    """docs/config-reference.md is generated from the configuration dataclasses: regenerate it when a key is added."""
    import os

    from primus_b200.tools import config_reference

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "docs", "config-reference.md")
    assert open(path).read() == config_reference.render(), "run: python -m primus_b200.tools.config_reference > docs/config-reference.md"
