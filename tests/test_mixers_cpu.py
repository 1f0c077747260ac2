"""Sequence mixers other than attention: Mamba-2 (state-space duality) and the LFM2 gated short convolution, checked
against step-by-step recurrences, torch's convolution and the Hugging Face implementations of both architectures."""
import pytest
import torch

from primus_b200.models import mixers as M
from primus_b200.models.config import TransformerConfig, hybrid_layer_pattern


@pytest.mark.parametrize("l,chunk", [(37, 8), (64, 16), (5, 8)])
def test_chunked_state_space_scan_matches_the_recurrence(l, chunk):
    torch.manual_seed(0)
    b, h, p, g, n = 2, 4, 8, 2, 16
    x = torch.randn(b, l, h, p)
    dt = torch.rand(b, l, h) * 0.5 + 0.01
    A = -torch.rand(h) * 2 - 0.1
    B, C = torch.randn(b, l, g, n), torch.randn(b, l, g, n)
    y1, y2 = M.ssd_chunked(x, dt, A, B, C, chunk), M.ssd_sequential(x, dt, A, B, C)
    assert (y1 - y2).abs().max() <= 1e-4 * y2.abs().max()


def test_causal_depthwise_convolution_matches_torch_and_does_not_cross_sequences():
    torch.manual_seed(1)
    x, w, bias = torch.randn(2 * 10, 6), torch.randn(6, 3), torch.randn(6)
    out = M.causal_depthwise_conv(x, w, bias, 2)
    ref = torch.nn.functional.conv1d(x.view(2, 10, 6).transpose(1, 2), w[:, None, :], bias, padding=2, groups=6)
    assert torch.allclose(out, ref[..., :10].transpose(1, 2).reshape(20, 6), atol=1e-6)
    x2 = x.clone()
    x2[:10] += 1.0                                   # the first sequence changes: the second one's output must not
    assert torch.equal(M.causal_depthwise_conv(x2, w, bias, 2)[10:], out[10:])


def test_hybrid_layer_pattern():
    assert hybrid_layer_pattern(8, 0.0, 0.0, hybrid=False) == "M" * 8
    assert hybrid_layer_pattern(8, 0.0, 0.0) == "M-" * 4
    p = hybrid_layer_pattern(32, 0.25, 0.0)             # mixers alternate with MLP layers; every fourth mixer is attention
    assert p == "*-M-M-M-" * 4
    assert hybrid_layer_pattern(12, 0.75, 0.0) == "*-*-*-M-*-M-" and hybrid_layer_pattern(10, 0.4, 0.0) == "*-M-*-M-M-"
    q = hybrid_layer_pattern(16, 0.125, 0.5)
    assert q.count("*") == 2 and q.count("-") == 8 and q.count("M") == 6
    assert hybrid_layer_pattern(4, 0.5, 0.0, "M*|-M") == "M*-M"
    with pytest.raises(AssertionError):
        hybrid_layer_pattern(4, 0, 0, "M*x-")
    cfg = TransformerConfig(num_layers=4, model_type="mamba", is_hybrid_model=True, hybrid_override_pattern="M*-M",
                            hidden_size=64, mamba_head_dim=16, mamba_num_groups=2, mamba_state_dim=16)
    assert cfg.layer_kinds == [("mamba", False), ("attention", False), (None, True), ("mamba", False)]


def _engine(cfg_kwargs, hf_sd, tokens):
    from primus_b200.engine import hf_convert as H
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    cfg = TransformerConfig(**dict(cfg_kwargs, params_dtype="fp32", seq_length=tokens.shape[1],
                                   make_vocab_size_divisible_by=8))
    model = GPTModel(cfg, "cpu")
    sd = H.hf_to_internal({k: v.detach().clone() for k, v in hf_sd.items()}, cfg)
    missing = [k for k in model.state_dict() if k not in sd]
    assert not missing, missing
    model.load_state_dict(sd, strict=True)
    n_params = sum(p.numel() for p in model.parameters())
    assert n_params == cfg.num_parameters(), (n_params, cfg.num_parameters())
    with torch.no_grad():
        return model(tokens)[:, : cfg.vocab_size]


def test_mamba2_matches_hf():
    T = pytest.importorskip("transformers.models.mamba2")
    from primus_b200.engine import hf_convert as H

    torch.manual_seed(0)
    # one group: the Hugging Face fallback path normalises the gated output over the whole inner dimension, Megatron's
    # mixer (followed here) over each group's share; with a single group the two definitions coincide
    c = T.Mamba2Config(vocab_size=250, hidden_size=64, state_size=16, num_hidden_layers=2, head_dim=16, num_heads=8,
                       n_groups=1, expand=2, conv_kernel=4, chunk_size=8, tie_word_embeddings=True, use_bias=False,
                       use_conv_bias=True, rms_norm=True, residual_in_fp32=False)
    m = T.Mamba2ForCausalLM(c).eval()
    for n, p in m.named_parameters():
        if n.endswith(("conv1d.bias", "mixer.norm.weight", "D")):
            torch.nn.init.normal_(p, mean=1.0, std=0.3)
    tokens = torch.randint(0, 250, (2, 21))
    with torch.no_grad():
        ref = m(tokens).logits.reshape(-1, 250)
    got = _engine(H.mamba2_config_from_hf(c.to_dict()), m.state_dict(), tokens)
    assert (got - ref).abs().max() <= 3e-4 * max(1.0, ref.abs().max().item())


def test_lfm2_matches_hf():
    T = pytest.importorskip("transformers.models.lfm2")
    from primus_b200.engine import hf_convert as H

    torch.manual_seed(1)
    c = T.Lfm2Config(vocab_size=250, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, max_position_embeddings=128,
                     layer_types=["conv", "full_attention", "conv"], conv_L_cache=3, conv_bias=False,
                     block_auto_adjust_ff_dim=False, tie_word_embeddings=True)
    m = T.Lfm2ForCausalLM(c).eval()
    tokens = torch.randint(0, 250, (2, 24))
    with torch.no_grad():
        ref = m(tokens).logits.reshape(-1, 250)
    kw = H.config_from_hf(c.to_dict())
    got = _engine(kw, m.state_dict(), tokens)
    assert (got - ref).abs().max() <= 3e-4 * max(1.0, ref.abs().max().item())


def test_hybrid_stack_trains_on_cpu():
    """Mamba + attention + MLP layers in one stack: the loss falls on a learnable synthetic stream."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=6, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                           vocab_size=256, params_dtype="fp32", model_type="mamba", is_hybrid_model=True,
                           hybrid_override_pattern="M-*-M-", mamba_head_dim=16, mamba_num_groups=2, mamba_state_dim=16,
                           mamba_chunk_size=16, untie_embeddings_and_output_weights=False)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=32, train_iters=12, lr=5e-3,
                     lr_decay_style="constant", mock_data_kind="markov")
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    losses = tr.train()
    assert losses[-1] < losses[0] - 0.1, losses
    ps.destroy_model_parallel()


@pytest.mark.parametrize("l,chunk", [(37, 8), (64, 16), (5, 8)])
def test_chunked_gated_delta_rule_matches_the_recurrence_and_hf(l, chunk):
    torch.manual_seed(2)
    b, h, dk, dv = 2, 3, 8, 16
    q = torch.nn.functional.normalize(torch.randn(b, l, h, dk), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(b, l, h, dk), dim=-1)
    v, g, beta = torch.randn(b, l, h, dv), -torch.rand(b, l, h) * 0.5, torch.rand(b, l, h)
    seq = M.gated_delta_rule_sequential(q, k, v, g, beta)
    chk = M.gated_delta_rule_chunked(q, k, v, g, beta, chunk)
    assert (seq - chk).abs().max() <= 1e-5 * max(1.0, seq.abs().max().item())
    try:
        from transformers.models.qwen3_next.modeling_qwen3_next import torch_recurrent_gated_delta_rule as hf_rule
    except Exception:  # noqa: BLE001
        return
    ref, _ = hf_rule(q, k, v, g, beta, None, False, use_qk_l2norm_in_kernel=False)
    assert (ref.float() - seq).abs().max() <= 1e-5


def test_gated_delta_rule_gradients_match_the_recurrence():
    torch.manual_seed(3)
    b, l, h, dk, dv = 1, 19, 2, 4, 6
    base = [torch.nn.functional.normalize(torch.randn(b, l, h, dk), dim=-1), torch.nn.functional.normalize(torch.randn(b, l, h, dk), dim=-1),
            torch.randn(b, l, h, dv), -torch.rand(b, l, h) * 0.3, torch.rand(b, l, h)]
    grads = []
    for fn in (M.gated_delta_rule_sequential, lambda *a: M.gated_delta_rule_chunked(*a, 8)):
        xs = [t.clone().requires_grad_() for t in base]
        fn(*xs).pow(2).sum().backward()
        grads.append([x.grad for x in xs])
    for a, c in zip(*grads):
        assert (a - c).abs().max() <= 1e-4 * max(1.0, a.abs().max().item())


def test_gated_delta_net_stack_trains_and_counts_parameters():
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                           vocab_size=256, params_dtype="fp32", model_type="mamba", is_hybrid_model=True,
                           linear_attention_type="gdn", hybrid_override_pattern="M-*-", linear_num_key_heads=2,
                           linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_chunk_size=16,
                           untie_embeddings_and_output_weights=False)
    assert mc.layer_kinds[0] == ("gdn", False)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=32, train_iters=12, lr=5e-3,
                     lr_decay_style="constant", mock_data_kind="markov")
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    assert sum(p.numel() for p in tr.model.parameters()) == mc.num_parameters()
    losses = tr.train()
    assert losses[-1] < losses[0] - 0.1, losses
    ps.destroy_model_parallel()


def test_qwen3_5_style_stack_trains_and_resumes(tmp_path):
    """Linear-attention layers inside a GPT-style stack (``linear_attention_freq``), gated attention output, zero-centred
    norm gains and a gated shared expert through the trainer and a checkpoint round trip."""
    from primus_b200.engine.trainer import Trainer
    from primus_b200.ops import fused
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    extra = dict(experimental_attention_variant="gated_delta_net", linear_attention_freq=2, linear_num_key_heads=2,
                 linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_chunk_size=16,
                 attention_output_gate=True, apply_layernorm_1p=True, rotary_percent=0.5, qk_layernorm=True,
                 moe_shared_expert_intermediate_size=32, moe_shared_expert_gate=True)

    def make(iters):
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, layers=4, moe=True, extra_mc=extra)
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        return Trainer(mc, tc, device="cpu", log_fn=lambda s: None)

    try:
        tr = make(4)
        assert [k for k, _ in tr.mcfg.layer_kinds] == ["gdn", "attention", "gdn", "attention"]
        gains = [p for n, p in tr.model.named_parameters() if n.endswith("layer_norm_weight")]
        assert gains and all(float(p.detach().abs().max()) == 0.0 for p in gains)          # stored as gain - 1
        losses = tr.train()
        assert len(losses) == 4 and all(x == x and abs(x) < 1e3 for x in losses)
        assert any(float(p.detach().abs().max()) > 0.0 for p in gains)                      # and trained
        tr.tcfg.save = str(tmp_path)
        tr.save_checkpoint()
        tr2 = make(6)
        assert tr2.load_checkpoint(str(tmp_path)) == 4
        for (n, a), (_, b) in zip(tr.model.named_parameters(), tr2.model.named_parameters()):
            assert torch.equal(a, b), n
    finally:
        fused.set_zero_centered_gamma(False)
        ps.destroy_model_parallel()
