"""Named random streams (tensor-parallel aware dropout), their replay under activation recompute and in checkpoints."""
import json

import pytest
import torch

from primus_b200.parallel import random as prandom
from tests.mp_utils import run_ranks


def test_streams_are_independent_and_leave_the_default_generator_alone():
    torch.manual_seed(7)
    before = torch.get_rng_state().clone()
    prandom.model_parallel_manual_seed(123, "cpu", tp_rank=1, pp_rank=2)
    t = prandom.get_rng_tracker()
    assert torch.equal(torch.get_rng_state(), before)
    assert t.seeds == {prandom.DATA_PARALLEL: 323, prandom.MODEL_PARALLEL: 123 + 2718 + 1 + 200,
                       prandom.EXPERT_PARALLEL: 123 + 1024 + 1}
    with t.fork(prandom.MODEL_PARALLEL):
        a = torch.rand(4)
    assert torch.equal(torch.get_rng_state(), before)        # the region did not consume default numbers
    with t.fork(prandom.MODEL_PARALLEL):
        b = torch.rand(4)
    assert not torch.equal(a, b)                              # the stream advances
    prandom.model_parallel_manual_seed(123, "cpu", tp_rank=1, pp_rank=2)
    with prandom.get_rng_tracker().fork(prandom.MODEL_PARALLEL):
        assert torch.equal(torch.rand(4), a)                  # and is reproducible from its seed
    with pytest.raises(ValueError):
        prandom.get_rng_tracker().add("again", 323)           # a seed may serve one stream only
    with pytest.raises(KeyError):
        with prandom.get_rng_tracker().fork("nope"):
            pass
    prandom.get_rng_tracker().reset()


def test_tensor_parallel_ranks_share_the_replicated_stream_only():
    masks = {}
    for tp_rank in (0, 1):
        prandom.model_parallel_manual_seed(5, "cpu", tp_rank=tp_rank)
        x = torch.ones(64)
        masks[tp_rank] = (prandom.dropout(x, 0.5, True, sharded=False), prandom.dropout(x, 0.5, True, sharded=True))
    assert torch.equal(masks[0][0], masks[1][0])
    assert not torch.equal(masks[0][1], masks[1][1])
    assert prandom.dropout(x, 0.5, False, True) is x and prandom.dropout(x, 0.0, True, True) is x
    prandom.get_rng_tracker().reset()


def test_recompute_replays_the_dropout_mask():
    prandom.model_parallel_manual_seed(11, "cpu")
    w = torch.randn(16, 16, requires_grad=True)
    x = torch.randn(8, 16)

    def block(h):
        return prandom.dropout(torch.tanh(h @ w), 0.5, True, sharded=True)

    states = prandom.get_rng_tracker().get_states()
    y = block(x).sum()
    y.backward()
    g_plain, w.grad = w.grad.clone(), None
    after_plain = prandom.get_rng_tracker().get_states()
    prandom.get_rng_tracker().set_states(states)
    y2 = prandom.checkpoint(block, x).sum()
    # something else draws from the stream between forward and backward
    prandom.dropout(torch.ones(4), 0.5, True, True)
    later = prandom.get_rng_tracker().get_states()
    y2.backward()
    assert torch.equal(y, y2) and torch.equal(w.grad, g_plain)
    now = prandom.get_rng_tracker().get_states()
    assert all(torch.equal(now[k], later[k]) for k in now)     # the recomputation left the streams where they were
    assert not torch.equal(later[prandom.MODEL_PARALLEL], after_plain[prandom.MODEL_PARALLEL])
    prandom.get_rng_tracker().reset()


def _train(kw, iters, tmp, resume_from=None, save_at=None):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    mc, tc = W.tiny_cfgs(**kw)
    tc.train_iters = iters
    if save_at is not None:
        tc.save, tc.save_interval = str(tmp), save_at
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    if resume_from is not None:
        assert tr.load_checkpoint(str(resume_from)) == 2
    out = tr.train()
    ps.destroy_model_parallel()
    return out


def test_hidden_dropout_changes_training_is_reproducible_and_resumes_bit_exactly(tmp_path):
    base = dict(seq=32, gbs=4, mbs=2, iters=4, layers=2)
    plain = _train(base, 4, tmp_path)
    kw = dict(base, extra_mc=dict(hidden_dropout=0.2))
    a = _train(kw, 4, tmp_path)
    b = _train(kw, 4, tmp_path)
    assert a == b and a != plain
    # full recompute replays the masks: same trajectory as without recompute
    c = _train(dict(base, extra_mc=dict(hidden_dropout=0.2, recompute_granularity="full", recompute_method="uniform",
                                        recompute_num_layers=1)), 4, tmp_path)
    assert all(abs(x - y) < 1e-5 for x, y in zip(a, c)), (a, c)
    # resume in the middle: the named streams come back from the checkpoint
    _train(kw, 2, tmp_path / "ck", save_at=2)
    d = _train(kw, 4, tmp_path, resume_from=tmp_path / "ck")
    assert d == a[2:], (a, d)


def _tp_worker(rank, world, kw, outp):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    mc, tc = W.tiny_cfgs(**kw)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(tp=mc.tensor_model_parallel_size)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    losses = tr.train()
    checksum = float(sum(p.float().abs().sum() for n, p in tr.model.named_parameters() if "layernorm" in n or "layer_norm" in n))
    with open(f"{outp}.{rank}", "w") as f:
        json.dump({"losses": losses, "norm_checksum": checksum}, f)


def test_replicated_dropout_keeps_tensor_parallel_ranks_in_step(tmp_path):
    """Without sequence parallelism the dropped activations are replicated: both ranks must draw the same mask, or
    their replicated norm weights would drift apart."""
    kw = dict(seq=32, gbs=4, mbs=2, iters=3, layers=2, tp=2, sp=False, extra_mc=dict(hidden_dropout=0.3))
    outp = str(tmp_path / "tp")
    run_ranks(_tp_worker, 2, "gloo", args=(kw, outp), timeout=240)
    r0, r1 = (json.load(open(f"{outp}.{r}")) for r in (0, 1))
    assert r0["losses"] == r1["losses"]
    assert r0["norm_checksum"] == r1["norm_checksum"]
