"""Host-side choices of the fused tensor-parallel kernels (no GPU needed)."""


def test_fused_tp_copy_cta_model():
    """Link-bound shapes (small GEMM per gathered / reduced byte) get more copy CTAs than compute-bound ones; TP = 2 and
    an explicit environment setting keep the default."""
    from primus_b200.parallel import fused_tp

    class Ctx:
        tp = 8

    class Inst:
        M = 8192

    def pick(mode, N, K, tp=8):
        Ctx.tp, Inst.mode, Inst.N, Inst.K = tp, mode, N, K
        return fused_tp._comm_ctas(Ctx, Inst)

    assert pick(0, 1280, 8192) > pick(0, 7168, 8192) >= 8          # QKV vs FC1 all-gather
    assert pick(1, 8192, 1024) > pick(1, 8192, 3584)               # projection vs FC2 reduce-scatter
    assert pick(1, 8192, 1024) % 8 == 0 and pick(1, 8192, 1024) <= 48
    assert pick(1, 8192, 4096, tp=2) == fused_tp.COMM_CTAS


def test_tp_pp_dp_rank_order():
    """``use_tp_pp_dp_mapping``: the stages of a pipeline sit on neighbouring ranks, data-parallel replicas far apart."""
    from primus_b200.parallel import state as ps

    world, tp, cp, pp = 16, 2, 1, 2
    a = ps.group_rank_lists(world, tp, cp, pp)
    b = ps.group_rank_lists(world, tp, cp, pp, tp_pp_dp=True)
    assert a["pp"][0] == [0, 8] and b["pp"][0] == [0, 2]
    assert a["dp"][0] == [0, 2, 4, 6] and b["dp"][0] == [0, 4, 8, 12]
    assert a["tp"][0] == b["tp"][0] == [0, 1]
    for lists in (a, b):        # every kind of group partitions the ranks
        for kind in ("tp", "dp", "pp", "ep", "edp"):
            assert sorted(r for g in lists[kind] for r in g) == list(range(world)), kind
    for r in range(world):
        t, c, d, p = ps.rank_coords(r, tp, cp, world // (tp * cp * pp), pp, tp_pp_dp=True)
        assert r in b["tp"][[g[0] for g in b["tp"]].index(r - t)] and b["stage"][p].count(r) == 1
        assert b["pp"][[i for i, g in enumerate(b["pp"]) if r in g][0]].index(r) == p
        assert b["dp"][[i for i, g in enumerate(b["dp"]) if r in g][0]].index(r) == d
    # expert groups tile every stage whatever the order of the ranks
    e = ps.group_rank_lists(16, 1, 1, 2, ep=4, tp_pp_dp=True)
    assert all(len({ps.rank_coords(r, 1, 1, 8, 2, True)[3] for r in g}) == 1 for g in e["ep"])
