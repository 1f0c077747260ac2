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
