"""GEMM tile-configuration cache: keys, shape dump, offline tuning with a fake timer, table files, environment policy."""
import json
import os

import pytest

from primus_b200.ops import autotune


@pytest.fixture(autouse=True)
def _clean(monkeypatch):
    autotune.clear()
    autotune.record_shapes(False)
    autotune.set_online(False)
    monkeypatch.setattr(autotune, "_TIMER", None)
    yield
    autotune.clear()
    autotune.record_shapes(False)
    autotune.set_online(False)


def test_candidates_depend_on_kind_and_shape():
    k = autotune.make_key("mxfp8", 8192, 4096, 4096, False, False, 0)
    assert autotune.candidates(k) == [{"block_n": 256}, {"block_n": 128}, {"two_cta": True}]
    assert autotune.candidates(autotune.make_key("bf16", 8192, 4096, 4096, False, False, 0)) == [{"block_n": 256}, {"block_n": 128}]
    assert autotune.candidates(autotune.make_key("mxfp8", 128, 128, 256, True, True, 2)) == [{"block_n": 128}]
    assert autotune.candidates(autotune.make_key("mxfp8", 384, 512, 256, False, False, 0))[-1] == {"block_n": 128}  # M % 256


def test_three_stage_workflow_with_a_fake_timer(tmp_path, monkeypatch):
    a = autotune.make_key("mxfp8", 8192, 6144, 4096, False, False, 0)
    b = autotune.make_key("bf16", 4096, 4096, 8192, True, True, 2)
    # stage 1: record
    assert not autotune.active()
    autotune.record_shapes(True)
    assert autotune.active()
    for _ in range(3):
        assert autotune.lookup(a) is None
    autotune.lookup(b)
    p1 = autotune.dump_shapes(str(tmp_path / "gemm_shape" / "r0.json"))
    p2 = str(tmp_path / "gemm_shape" / "r1.json")
    json.dump({"version": 1, "shapes": {"mxfp8:8192:6144:4096:0:0:0": 5}}, open(p2, "w"))
    seen = autotune.read_shapes([p1, p2])
    assert seen == {a: 8, b: 1}
    autotune.record_shapes(False)
    # stage 2: tune (the fake timer prefers the CTA pair for a, the 128-wide tile for b)
    monkeypatch.setattr(autotune, "_TIMER", lambda key, o: {"two_cta": 1e-3}.get(next(iter(o)), 2e-3)
                        if key == a else (1e-3 if o.get("block_n") == 128 else 3e-3))
    lines = []
    autotune.tune_shapes(seen, log=lines.append)
    assert autotune.lookup(a)["two_cta"] is True and autotune.lookup(b)["block_n"] == 128
    assert autotune.lookup(a)["time_us"] == 1000.0 and len(autotune.lookup(a)["candidates_us"]) == 3 and len(lines) == 2
    out = str(tmp_path / "gemm_tune" / "tuned.json")
    autotune.save(out)
    # stage 3: a fresh process loads the file
    autotune.clear()
    assert autotune.lookup(a) is None
    assert autotune.load(out) == 2
    assert autotune.lookup(a)["two_cta"] is True
    assert autotune.lookup(autotune.make_key("bf16", 1, 2, 3, False, False, 0)) is None      # unknown keys: heuristic


def test_online_mode_tunes_on_first_use_and_deterministic_mode_switches_everything_off(monkeypatch):
    calls = []
    monkeypatch.setattr(autotune, "_TIMER", lambda key, o: calls.append(o) or (1.0 if o.get("block_n") == 256 else 0.5))
    k = autotune.make_key("bf16", 1024, 1024, 1024, False, False, 0)
    autotune.set_online(True)
    assert autotune.lookup(k)["block_n"] == 128 and len(calls) == 2
    assert autotune.lookup(k)["block_n"] == 128 and len(calls) == 2          # cached
    monkeypatch.setenv("PRIMUS_DETERMINISTIC", "1")
    assert autotune.lookup(k) is None
    autotune.set_online(True)
    assert not autotune._ONLINE


def test_a_rejected_candidate_is_skipped(monkeypatch):
    def timer(key, o):
        if o.get("two_cta"):
            raise RuntimeError("not supported")
        return 1.0 if o["block_n"] == 256 else 2.0

    monkeypatch.setattr(autotune, "_TIMER", timer)
    k = autotune.make_key("mxfp8", 512, 512, 512, False, False, 0)
    r = autotune.tune_key(k)
    assert r["block_n"] == 256 and "rejected" in r["candidates_us"]['{"two_cta": true}']


def test_gemm_consults_the_table_on_cpu_without_side_effects():
    """The CPU path of ops.gemm ignores tile options; recording still sees the call's key."""
    import torch

    from primus_b200.ops import gemm

    autotune.record_shapes(True)
    a, b = torch.randn(8, 16), torch.randn(4, 16)
    out = gemm.gemm(a, b)
    assert torch.allclose(out, a @ b.t(), atol=1e-5)
    # the CPU path returns before the launch options are needed: nothing is recorded for it
    assert autotune.seen_shapes() == {}


def test_model_shapes_cover_the_three_gemms_of_every_linear_layer():
    from primus_b200.tools.tune_gemm import model_shapes

    keys = model_shapes("llama3.1_8B", 8192, kinds=("mxfp8",))
    assert autotune.make_key("mxfp8", 8192, 6144, 4096, False, False, 0) in keys
    assert autotune.make_key("mxfp8", 8192, 4096, 6144, False, True, 0) in keys
    assert autotune.make_key("mxfp8", 6144, 4096, 8192, True, True, 2) in keys
    assert autotune.make_key("mxfp8", 8192, 28672, 4096, False, False, 0) in keys and len(keys) == 12
