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
