"""Activation recomputation: every mode must give the same loss and gradients as no recomputation, and must run the
layers again in the backward pass exactly where the mode says so."""
import dataclasses

import pytest
import torch

from primus_b200.models.config import TransformerConfig
from primus_b200.models.gpt import GPTModel, recompute_plan
from primus_b200.parallel import state as ps


def _cfg(**kw):
    return TransformerConfig(num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                             vocab_size=256, params_dtype="fp32", make_vocab_size_divisible_by=64, seq_length=16, **kw)


def _run(cfg):
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(3)
    m = GPTModel(cfg, "cpu")
    calls = {i: 0 for i in range(cfg.num_layers)}
    for i in range(cfg.num_layers):
        m.decoder.layers[str(i)].register_forward_pre_hook(lambda mod, a, i=i: calls.__setitem__(i, calls[i] + 1))
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, 256, (2, 16), generator=g)
    lab = torch.randint(0, 256, (2, 16), generator=g)
    w = torch.full((2, 16), 1.0 / 32)
    loss = m(tok, lab, loss_weights=w)
    loss.backward()
    grads = {n: (p.grad if p.grad is not None else p.main_grad).detach().clone() for n, p in m.named_parameters()
             if p.grad is not None or getattr(p, "main_grad", None) is not None}
    ps.destroy_model_parallel()
    return float(loss.detach()), grads, calls


MODES = {
    "uniform_1": (dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=1), [2, 2, 2, 2]),
    "uniform_2": (dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2), [2, 2, 2, 2]),
    "uniform_3": (dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=3), [2, 2, 2, 2]),
    "block_1": (dict(recompute_granularity="full", recompute_method="block", recompute_num_layers=1), [2, 1, 1, 1]),
    "block_3": (dict(recompute_granularity="full", recompute_method="block", recompute_num_layers=3), [2, 2, 2, 1]),
    "layer_ids": (dict(recompute_granularity="full", recompute_layer_ids=[1, 3]), [1, 2, 1, 2]),
    "full_default": (dict(recompute_granularity="full"), [2, 2, 2, 2]),
    "selective": (dict(recompute_granularity="selective"), [1, 1, 1, 1]),
    "selective_mlp": (dict(recompute_granularity="selective", recompute_modules=["core_attn", "mlp"]), [1, 1, 1, 1]),
}


@pytest.mark.parametrize("name", sorted(MODES))
def test_recompute_modes_match_plain_run(name):
    kw, expected_calls = MODES[name]
    ref_loss, ref_grads, ref_calls = _run(_cfg())
    assert list(ref_calls.values()) == [1, 1, 1, 1]
    loss, grads, calls = _run(_cfg(**kw))
    assert abs(loss - ref_loss) < 1e-6
    assert list(calls.values()) == expected_calls, calls
    assert grads.keys() == ref_grads.keys()
    for n in grads:
        assert torch.allclose(grads[n], ref_grads[n], rtol=1e-5, atol=1e-7), n


def test_plan_groups():
    cfg = _cfg(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=3)
    assert recompute_plan(cfg, [4, 5, 6, 7, 8]) == [([4, 5, 6], True), ([7, 8], True)]
    cfg = _cfg(recompute_granularity="full", recompute_method="block", recompute_num_layers=2)
    assert recompute_plan(cfg, [4, 5, 6]) == [([4], True), ([5], True), ([6], False)]
    with pytest.raises(ValueError):
        recompute_plan(_cfg(recompute_granularity="full", recompute_method="nope"), [0])


def test_selective_recomputes_core_attention_only(monkeypatch):
    """Under selective recomputation the core attention runs twice per layer (forward + backward), nothing else does."""
    from primus_b200.ops import layers

    n = {"attn": 0}
    real = layers.rope_attention

    def counted(*a, **k):
        n["attn"] += 1
        return real(*a, **k)

    monkeypatch.setattr(layers, "rope_attention", counted)
    _run(_cfg())
    assert n["attn"] == 4
    n["attn"] = 0
    _run(_cfg(recompute_granularity="selective"))
    assert n["attn"] == 8
