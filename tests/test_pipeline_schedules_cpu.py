"""Schedule-table invariants: every micro-batch has F and B on every stage, F precedes B, zero-bubble splits B into
B + W, tables execute without deadlock, and bubble fractions order as expected."""
import pytest

from primus_b200.parallel import pipeline_schedules as S

ALGOS = ["1f1b", "interleaved", "zerobubble", "zbv", "v-half", "v-min"]


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("pp,m", [(2, 4), (4, 8), (4, 4), (8, 16)])
def test_tables_are_complete_and_executable(algo, pp, m):
    sch = S.build_schedule(algo, pp, m, vpp=2)
    S.validate(sch["table"], pp, m, sch["chunks"], sch["placement"])
    kinds = {n.kind for seq in sch["table"] for n in seq}
    if algo in ("zerobubble", "zbv", "v-half", "v-min"):
        assert "W" in kinds and "B" in kinds and "BW" not in kinds
    else:
        assert kinds == {"F", "BW"}


def test_1f1b_shape():
    t = S.schedule_1f1b(4, 8)
    assert [n.kind for n in t[0][:3]] == ["F", "F", "F"] and t[0][3].kind == "F" and t[0][4].kind == "BW"
    assert [n.kind for n in t[3][:2]] == ["F", "BW"]
    for r in range(4):
        assert sum(n.kind == "F" for n in t[r]) == 8 and sum(n.kind == "BW" for n in t[r]) == 8


def test_interleaved_warmup_and_constraints():
    pp, vpp, m = 4, 2, 8
    t = S.schedule_interleaved(pp, vpp, m)
    for r in range(pp):
        warm = 0
        for n in t[r]:
            if n.kind != "F":
                break
            warm += 1
        assert warm == min((pp - r - 1) * 2 + (vpp - 1) * pp, m * vpp) + 1 or warm == (pp - r - 1) * 2 + (vpp - 1) * pp + 1
    with pytest.raises(ValueError):
        S.schedule_interleaved(4, 2, 6)


def test_bubble_ordering():
    pp, m = 4, 8
    res = {}
    for algo in ("1f1b", "interleaved", "zerobubble", "zbv"):
        sch = S.build_schedule(algo, pp, m, vpp=2 if algo == "interleaved" else None)
        c = sch["chunks"]
        res[algo] = S.simulate(sch["table"], pp, c, sch["placement"], 1.0 / c, 1.0 / c, 1.0 / c)["bubble_fraction"]
    assert res["interleaved"] < res["1f1b"]
    assert res["zerobubble"] < res["1f1b"]
    assert res["zbv"] <= res["zerobubble"] + 1e-6
    expected = (pp - 1) / (m + pp - 1)  # classic 1F1B bubble with t_b = 2 t_f
    assert abs(res["1f1b"] - expected) < 1e-6


def test_comm_expansion_v_fold_has_no_comm_on_the_fold():
    sch = S.build_schedule("zbv", 4, 4)
    full = S.expand_with_comm(sch["table"], 4, 2, "v")
    last = full[3]  # rank 3 holds stage 3 (chunk 0) and stage 4 (chunk 1): hand-off is local
    assert not any(n.kind == "SF" and n.chunk == 0 for n in last)
    assert not any(n.kind == "RF" and n.chunk == 1 for n in last)
    first = full[0]
    assert any(n.kind == "SF" and n.chunk == 0 for n in first) and any(n.kind == "RF" and n.chunk == 1 for n in first)


def test_pipeline_timeline_dump_and_viewer(tmp_path):
    """Timeline files written by the runtime are merged into a chart, bubble fractions and a Chrome trace."""
    import json

    from primus_b200.parallel.pipeline import PipelineTimeline
    from primus_b200.parallel.pipeline_schedules import Node
    from primus_b200.tools import pp_vis

    for r in range(2):
        tl = PipelineTimeline()
        for i in range(3):
            tl.add(Node("F", i, 0), r * 0.1 + i * 0.2, r * 0.1 + i * 0.2 + 0.1)
            tl.add(Node("B", i, 0), 1 + (1 - r) * 0.1 + i * 0.3, 1 + (1 - r) * 0.1 + i * 0.3 + 0.2)
        tl.dump(str(tmp_path / f"pp_rank{r}_iter3.json"), r, 3, {"schedule": "1f1b", "pp": 2})
    lines, bubbles = pp_vis.main([str(tmp_path), "--width", "60", "--trace", str(tmp_path / "t.json")])
    assert len(lines) == 2 and all(0.3 < b < 0.7 for b in bubbles.values())
    assert "F" in lines[0] and "B" in lines[1]
    trace = json.loads((tmp_path / "t.json").read_text())
    assert len(trace["traceEvents"]) == 12
