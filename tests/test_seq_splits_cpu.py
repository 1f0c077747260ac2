"""Sequence splits (``num_seq_splits``): a micro-batch processed as consecutive sequence chunks, with attention over the
kept keys / values of the earlier chunks, must give the losses and gradients of the unsplit run."""
import pytest
import torch

from primus_b200.engine.trainer import Trainer
from primus_b200.parallel import state as ps
from tests import dist_workers as W


def _run(splits, iters=3, **kw):
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, layers=2, extra_tc=dict(num_seq_splits=splits), **kw)
    torch.manual_seed(0)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    norms = []
    losses = tr.train(on_step=lambda t, lv: norms.append(float(t.optimizer.grad_norm.item())))
    ps.destroy_model_parallel()
    return losses, norms


@pytest.mark.parametrize("splits", [2, 4])
def test_chunked_sequence_matches_the_whole_sequence(splits):
    ref, ref_norms = _run(1)
    got, norms = _run(splits)
    assert all(abs(a - b) <= 1e-4 * max(1.0, abs(a)) for a, b in zip(ref, got)), (ref, got)
    assert all(abs(a - b) <= 2e-3 * max(1e-3, abs(a)) for a, b in zip(ref_norms, norms)), (ref_norms, norms)


def test_kv_cache_is_released_and_unsupported_combinations_are_rejected():
    from primus_b200.ops import layers

    _run(2, iters=1)
    assert layers.SEQ_SPLIT.cache == {} and not layers.SEQ_SPLIT.active
    with pytest.raises(NotImplementedError):
        _run(2, iters=1, extra_mc=dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=1))
    with pytest.raises(AssertionError):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc, tc = W.tiny_cfgs(seq=30, gbs=4, mbs=2, iters=1, layers=2, extra_tc=dict(num_seq_splits=4))
        Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
