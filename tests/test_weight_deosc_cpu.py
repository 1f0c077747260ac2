"""MXFP4 weight de-oscillation: the quantise-dequantise map, the detector on a scripted oscillation, the optimizer hook on
sharded master weights and the checkpoint round trip.  Behaviour of the reference's runner
(primus/backends/megatron/core/optimizer/weight_deosc.py:386-510; tests/unit_tests/backends/megatron/test_weight_deosc.py)."""
import torch

from primus_b200.ops import fp8
from primus_b200.parallel import distributed as D
from primus_b200.parallel.weight_deosc import WeightDeOsc, WeightDeOscConfig, qdq_mxfp4


def test_qdq_matches_the_forward_quantiser_and_is_idempotent():
    torch.manual_seed(0)
    w = (torch.randn(128, 256) * 0.05).to(torch.bfloat16)
    q = fp8.quantize_mxfp8_ref(w, True, False, scaling="mxfp4", is_weight=True)
    ref = fp8.dequantize_mxfp8_ref(q.q_row.view(128, 256), q.sf_row, colwise=False)
    got = qdq_mxfp4(w.float())
    assert torch.equal(got, ref)
    assert torch.equal(qdq_mxfp4(got), got)                      # codes are fixed points
    assert torch.equal(qdq_mxfp4(w.float().view(-1)[64:64 + 96]), ref.view(-1)[64:64 + 96])   # block-aligned slices


def _one_bucket_optimizer(params, dp_size=1, dp_rank=0):
    buf = D.ParamGradBuffer(params, None, dp_size, dp_rank, use_distributed_optimizer=dp_size > 1)
    buf.use_distributed_optimizer = True            # shard ranges of rank ``dp_rank`` without a process group
    opt = D.DistributedOptimizer([buf], lr=1e-3, weight_decay=0.0, clip_grad=0.0)
    return buf, opt


def test_detector_snaps_only_the_oscillating_elements():
    torch.manual_seed(1)
    w = torch.nn.Parameter(torch.zeros(64, 64))
    with torch.no_grad():
        # block maximum 6 -> scale 1: the codes are the E2M1 grid itself, the boundary between 2 and 3 lies at 2.5
        w[:, 0] = 6.0
        w[:, 1] = 2.5 - 2e-2            # flips between the codes 2 and 3 under a tiny oscillation
        w[:, 2] = 1.2                   # drifts without changing its code for a while
    buf, opt = _one_bucket_optimizer([w])
    de = WeightDeOsc(WeightDeOscConfig(True, period=6, ratio_threshold=4.0), eligible=lambda p: True, log=lambda m: None)
    master = opt.state[0]["master"]
    o = buf.param_offsets[w]
    view = master[o:o + w.numel()].view(64, 64)
    closed = []
    for t in range(7):                   # the first call only seeds the window
        view[:, 1] = 2.5 + (2e-2 if t % 2 == 0 else -2e-2)
        view[:, 2] += 1e-3
        closed.append(de.run(opt))
    assert closed == [False] * 6 + [True]
    assert de.last_snapped == 64                         # the flipping column, nothing else
    assert torch.all((view[:, 1] == 2.0) | (view[:, 1] == 3.0))
    assert torch.allclose(view[:, 2], torch.full((64,), 1.207), atol=1e-5)
    assert torch.equal(buf.param_data[o:o + w.numel()].view(64, 64)[:, 1], view[:, 1])     # the parameter follows
    # after the snap the element sits on a code: the same perturbation no longer flips it
    for t in range(6):
        view[:, 1] += (2e-2 if t % 2 == 0 else -2e-2)
        de.run(opt)
    assert de.last_snapped == 0 and de.periods == 2


def test_ineligible_and_start_step():
    w = torch.nn.Parameter(torch.randn(32, 64))
    b = torch.nn.Parameter(torch.randn(64))                  # 1-D: never tracked
    odd = torch.nn.Parameter(torch.randn(32, 48))            # input dimension not a multiple of 32
    buf, opt = _one_bucket_optimizer([w, b, odd])
    de = WeightDeOsc(WeightDeOscConfig(True, period=2, start_step=3), eligible=lambda p: True, log=lambda m: None)
    de.run(opt); de.run(opt)
    assert de.last_tracked == 0
    de.run(opt)
    assert de.last_tracked == w.numel()


def test_shards_of_two_ranks_together_equal_the_unsharded_run():
    torch.manual_seed(2)
    shapes = [(64, 96), (32, 160), (96, 64)]
    init = [torch.randn(s) * 0.1 for s in shapes]

    def run(dp_size, dp_rank):
        params = [torch.nn.Parameter(t.clone()) for t in init]
        buf, opt = _one_bucket_optimizer(params, dp_size, dp_rank)
        de = WeightDeOsc(WeightDeOscConfig(True, period=4, ratio_threshold=2.0), eligible=lambda p: True,
                         log=lambda m: None)
        g = torch.Generator().manual_seed(3)
        st = opt.state[0]
        for t in range(5):
            noise = torch.randn(buf.numel, generator=g) * 3e-3      # the same walk for every layout
            st["master"] += noise[st["s"]:st["e"]]
            de.run(opt)
        full = torch.zeros(buf.numel)
        full[st["s"]:st["e"]] = st["master"]
        return full, de.last_snapped

    whole, n = run(1, 0)
    a, na = run(2, 0)
    b, nb = run(2, 1)
    assert n > 0 and na + nb == n
    assert torch.equal(a + b, whole)


def test_checkpoint_round_trip_continues_the_window():
    torch.manual_seed(4)
    init = torch.randn(64, 64) * 0.1

    def make():
        w = torch.nn.Parameter(init.clone())
        buf, opt = _one_bucket_optimizer([w])
        return opt, WeightDeOsc(WeightDeOscConfig(True, period=5, ratio_threshold=2.0), eligible=lambda p: True,
                                log=lambda m: None)

    g = torch.Generator().manual_seed(5)
    noise = [torch.randn(64 * 64, generator=g) * 3e-3 for _ in range(6)]
    opt, de = make()
    for t in range(6):
        opt.state[0]["master"][:4096] += noise[t]
        de.run(opt)
    ref, ref_n = opt.state[0]["master"].clone(), de.last_snapped

    opt, de = make()
    for t in range(3):
        opt.state[0]["master"][:4096] += noise[t]
        de.run(opt)
    sd, master = de.state_dict(), opt.state[0]["master"].clone()
    opt, de = make()
    opt.state[0]["master"].copy_(master)
    de.load_state_dict(sd)
    for t in range(3, 6):
        opt.state[0]["master"][:4096] += noise[t]
        de.run(opt)
    assert de.last_snapped == ref_n and ref_n > 0
    assert torch.equal(opt.state[0]["master"], ref)


def test_trainer_installs_the_detector_and_checkpoints_its_windows(tmp_path):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    def make(iters, extra_mc):
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, layers=2, extra_mc=extra_mc,
                             extra_tc=dict(weight_deosc=True, weight_deosc_period=2, weight_deosc_ratio=1.5))
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        logs = []
        tr = Trainer(mc, tc, device="cpu", log_fn=logs.append)
        return tr, logs

    try:
        tr, logs = make(1, {})
        assert tr.optimizer.deosc is None and any("fp4 is not" in m for m in logs)      # nothing is quantised to 4 bits
        tr, logs = make(5, dict(fp4="e2m1"))
        de = tr.optimizer.deosc
        assert de is not None and any("[weight de-osc] on" in m for m in logs)
        de.eligible = lambda p: True         # on a GPU the MXFP4 GEMMs mark the weights they quantise
        tr.train()
        assert de.global_step == 5 and de.periods == 2 and de.last_tracked > 0
        tr.tcfg.save = str(tmp_path)
        tr.save_checkpoint()
        tr2, _ = make(5, dict(fp4="e2m1"))
        tr2.optimizer.deosc.eligible = lambda p: True
        assert tr2.load_checkpoint(str(tmp_path)) == 5
        de2 = tr2.optimizer.deosc
        assert de2.global_step == 5 and de2.periods == 2 and set(de2._loaded) == set(de._windows)
        de2.run(tr2.optimizer)
        k = next(iter(de._windows))
        assert torch.equal(de2._windows[k].dist_w, torch.zeros_like(de2._windows[k].dist_w))   # no movement since
        assert de2._windows[k].step == de._windows[k].step + 1
    finally:
        gemm.set_fp8_recipe(None)
        ps.destroy_model_parallel()
