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
