"""Kimi-K3 building blocks against direct statements of their definitions: the delta-attention recurrence, attention
residuals, quantile balancing, the SiTU activation, the latent mixture of experts, NoPE multi-latent attention, and the
whole stack through the trainer.  The reference checks the same properties in
tests/unit_tests/megatron/transformer/kimi_k3/ (collapse to the gated delta rule, the un-normalised mixture, the
histogram quantile, the norm inside the latent bottleneck)."""
import math

import pytest
import torch
import torch.nn.functional as F

from primus_b200.models import kimi_k3 as K


def _qkvb(b=2, l=150, h=3, dk=16, dv=24, seed=0):
    torch.manual_seed(seed)
    q = F.normalize(torch.randn(b, l, h, dk), dim=-1)
    k = F.normalize(torch.randn(b, l, h, dk), dim=-1)
    return q, k, torch.randn(b, l, h, dv), torch.sigmoid(torch.randn(b, l, h))


@pytest.mark.parametrize("lower_bound", [None, -5.0, -60.0])
@pytest.mark.parametrize("chunk", [16, 64])
def test_chunked_delta_attention_matches_the_recurrence(lower_bound, chunk):
    q, k, v, beta = _qkvb()
    b, l, h, dk = q.shape
    g = K.kda_gate(torch.randn(b, l, h, dk) * 2, torch.randn(h) * 0.3, torch.randn(h * dk), lower_bound)
    assert g.max() <= 0 and (lower_bound is None or g.min() >= lower_bound)
    ref = K.kda_sequential(q, k, v, g, beta)
    out = K.kda_chunked(q, k, v, g, beta, chunk)
    assert torch.isfinite(out).all()                    # a decay of e^-60 per step overflows any 1 / decay formulation
    assert (out - ref).abs().max() < 2e-5


def test_channel_constant_gate_is_the_gated_delta_rule():
    from primus_b200.models.mixers import gated_delta_rule_sequential

    q, k, v, beta = _qkvb(seed=1)
    b, l, h, dk = q.shape
    g = -torch.rand(b, l, h) * 2
    ref = gated_delta_rule_sequential(q, k, v, g, beta)
    out = K.kda_chunked(q, k, v, g[..., None].expand(b, l, h, dk).contiguous(), beta, 64)
    assert (out - ref).abs().max() < 2e-5


def test_delta_attention_gradients_match_the_recurrence():
    q, k, v, beta = _qkvb(b=1, l=40, h=2, dk=8, dv=8, seed=2)
    g0 = K.kda_gate(torch.randn(1, 40, 2, 8), torch.zeros(2), None, -5.0)
    grads = []
    for fn in (K.kda_sequential, lambda *a: K.kda_chunked(*a, 16)):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g0, beta)]
        (fn(*leaves) * torch.arange(8).float()).sum().backward()
        grads.append([t.grad for t in leaves])
    for a, b_ in zip(*grads):
        assert (a - b_).abs().max() < 5e-5 * max(1.0, a.abs().max().item())


def test_attention_residual_mix():
    torch.manual_seed(3)
    T, n, H = 10, 3, 32
    stream, cps = torch.randn(T, H), torch.randn(T, n, H) * 3
    nw, pw = torch.rand(H) + 0.5, torch.randn(1, H)
    out = K.attn_res_mix(stream, cps, nw, pw, 1e-5)
    cand = torch.cat([cps, stream[:, None]], 1)
    normed = cand / cand.pow(2).mean(-1, keepdim=True).add(1e-5).sqrt()
    p = torch.softmax((normed * nw * pw[0]).sum(-1), -1)
    assert torch.allclose(out, (p[..., None] * cand).sum(1), atol=1e-5)       # the candidates themselves are mixed
    assert torch.allclose(K.attn_res_mix(stream, None, nw, pw, 1e-5), stream, atol=1e-6)      # one candidate: identity
    # scaling a candidate leaves its score alone (scores see the normalised form) but scales its share of the output
    out2 = K.attn_res_mix(stream, cps * torch.tensor([2.0, 1.0, 1.0])[None, :, None], nw, pw, 1e-5)
    assert torch.allclose(out2 - out, p[:, :1] * cps[:, 0], atol=1e-4)
    assert [K.checkpoints_before(i, 4) for i in range(8)] == [0, 1, 1, 1, 1, 2, 2, 2]


def test_histogram_quantile_and_balancing_bias():
    torch.manual_seed(4)
    x = torch.randn(5, 20000) * 0.2
    lo, hi, bins = -1.0, 1.0, 1024
    hist = torch.stack([torch.histc(r, bins, lo, hi) for r in x]).long()
    for q in (0.1, 0.5, 0.97):
        est = K.histogram_quantile(hist, q, lo, hi)
        assert (est.float() - torch.quantile(x, q, dim=1)).abs().max() < 2 * (hi - lo) / bins
    assert float(K.histogram_quantile(torch.zeros(1, bins).long(), 0.5, lo, hi)) == 0.0      # no counts: mid-range
    # skewed router: with the bias from the margins every expert gets close to its fair share of the tokens
    T, E, k = 8192, 16, 2
    scores = torch.sigmoid(torch.randn(T, E) + torch.linspace(-1.5, 1.5, E))
    bias = torch.zeros(E)

    def loads(b):
        return torch.bincount((scores + b).topk(k, -1).indices.reshape(-1), minlength=E).float()

    before = loads(bias)
    for _ in range(6):          # the cut-offs move with the bias: a few rounds approach the fixed point
        bias = K.quantile_bias(K.margin_histogram(scores, bias, k, bins, lo, hi), k, lo, hi).float()
    after = loads(bias)
    fair = T * k / E
    assert before.max() > 2.5 * fair and (after - fair).abs().max() < 0.15 * fair
    assert abs(float(bias.mean())) < 1e-6
    # the histogram holds every (token, expert) pair once; out-of-range margins land in the end bins
    h = K.margin_histogram(scores, bias, k, 8, -0.01, 0.01)
    assert h.sum() == T * E and h[:, 0].sum() > 0 and h[:, -1].sum() > 0


def test_situ_activation():
    from primus_b200.ops import fused

    x = torch.randn(7, 64) * 20
    g, u = x[:, :32], x[:, 32:]
    fused.set_situ_betas(4.0, 25.0)
    ref = 4.0 * torch.tanh(g / 4.0) * torch.sigmoid(g) * 25.0 * torch.tanh(u / 25.0)
    assert torch.allclose(fused.swiglu(x, None, 0.0, "situ"), ref, atol=1e-5)
    assert fused.swiglu(x, None, 0.0, "situ").abs().max() <= 100.0            # both factors are bounded
    small = torch.randn(7, 64) * 0.1
    assert torch.allclose(fused.swiglu(small, None, 0.0, "situ"), fused.swiglu(small, None, 0.0, "silu"), atol=1e-4)
    probs = torch.rand(7)
    assert torch.allclose(fused.swiglu(x, probs, 0.0, "situ"), ref * probs[:, None], atol=1e-5)


def _k3_cfg(**over):
    from primus_b200.models.config import TransformerConfig

    kw = dict(model_type="kimi_k3", num_layers=6, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4,
              kv_channels=16, vocab_size=256, params_dtype="fp32", q_lora_rank=32, kv_lora_rank=24, qk_head_dim=16,
              qk_pos_emb_head_dim=8, v_head_dim=16, mla_use_output_gate=True, linear_attention_freq="([1]*2+[0])*2",
              linear_num_key_heads=4, linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
              kda_chunk_size=32, attn_res_block_size=3, num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=32,
              moe_layer_freq="([0]*1+[1]*5)", moe_shared_expert_intermediate_size=64, routed_expert_hidden_size=32,
              moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True,
              moe_router_bias_update_rule="quantile", gated_activation="situ", untie_embeddings_and_output_weights=True)
    kw.update(over)
    return TransformerConfig(**kw)


def test_latent_moe_layer_matches_its_definition():
    from primus_b200.models.moe import MoELayer
    from primus_b200.ops import fused
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(5)
    cfg = _k3_cfg(moe_aux_loss_coeff=0.0)
    layer = MoELayer(cfg, 1, "cpu", 1)
    with torch.no_grad():
        layer.latent_norm.weight.uniform_(0.5, 1.5)
    y = torch.randn(24, 64)
    out = layer(y)
    w1, w2 = layer.experts.fc1_weight.weight, layer.experts.fc2_weight.weight
    assert w1.shape == (8, 64, 32) and w2.shape == (8, 32, 32)                 # experts live in the latent width
    scores = torch.sigmoid(y @ layer.router.weight.t())                        # the router reads the full-width input
    top = scores.topk(2, -1)
    probs = top.values / top.values.sum(-1, keepdim=True)
    x = y @ layer.fc1_latent_proj.weight.t()
    mix = torch.zeros(24, 32)
    for t in range(24):
        for j in range(2):
            e = int(top.indices[t, j])
            mix[t] += probs[t, j] * (fused.swiglu_ref((x[t] @ w1[e].t())[None], None, 0.0, "situ")[0] @ w2[e].t())
    mix = mix * torch.rsqrt(mix.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * layer.latent_norm.weight   # after the combine
    ref = mix @ layer.fc2_latent_proj.weight.t() + layer.shared_experts.forward_normed(y)    # shared experts: full width
    assert torch.allclose(out, ref, atol=2e-5)
    ps.destroy_model_parallel()


def test_nope_mla_ignores_positions_and_gates_its_output():
    from primus_b200.models.mla import MLASelfAttention
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(6)
    x = torch.randn(32, 64)

    def run(cfg, pos):
        torch.manual_seed(7)
        att = MLASelfAttention(cfg, 0, "cpu", 1)
        cos, sin = att.rope_tables("cpu", 64)
        return att, att(x, None, (cos, sin, pos, None), 1)[0]

    p0, p1 = torch.arange(32, dtype=torch.int32), (torch.arange(32, dtype=torch.int32) * 7) % 32
    _, a = run(_k3_cfg(), p0)
    att, b = run(_k3_cfg(), p1)
    assert torch.equal(a, b)                                                   # no rotation: positions do not enter
    _, c = run(_k3_cfg(model_type="gpt", multi_latent_attention=True, mla_use_output_gate=True), p0)
    _, d = run(_k3_cfg(model_type="gpt", multi_latent_attention=True, mla_use_output_gate=True), p1)
    assert (c - d).abs().max() > 1e-3 * c.abs().max()                           # with rotation they do
    with torch.no_grad():       # a very negative gate closes the output
        att.linear_o_gate.weight.zero_()
    cos, sin = att.rope_tables("cpu", 64)
    half = att(x, None, (cos, sin, p0, None), 1)[0]                            # sigmoid(0) = 1/2 on every channel
    _, ungated = run(_k3_cfg(mla_use_output_gate=False), p0)
    assert torch.allclose(half, 0.5 * ungated, atol=1e-5)
    ps.destroy_model_parallel()


def test_kimi_k3_stack_trains_updates_its_bias_and_resumes(tmp_path):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    extra = {k: v for k, v in vars(_k3_cfg()).items() if k in (
        "model_type", "q_lora_rank", "kv_lora_rank", "qk_head_dim", "qk_pos_emb_head_dim", "v_head_dim",
        "mla_use_output_gate", "linear_attention_freq", "linear_num_key_heads", "linear_num_value_heads",
        "linear_key_head_dim", "linear_value_head_dim", "kda_chunk_size", "attn_res_block_size", "num_experts",
        "moe_router_topk", "moe_ffn_hidden_size", "moe_layer_freq", "moe_shared_expert_intermediate_size",
        "routed_expert_hidden_size", "moe_router_score_function", "moe_router_enable_expert_bias",
        "moe_router_bias_update_rule", "gated_activation")}

    def make(iters, **more):
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, layers=6, extra_mc=dict(extra, **more))
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        return Trainer(mc, tc, device="cpu", log_fn=lambda s: None)

    try:
        tr = make(3)
        kinds = [k for k, _ in tr.mcfg.layer_kinds]
        assert kinds == ["kda", "kda", "attention", "kda", "kda", "attention"]
        names = [n for n, _ in tr.model.named_parameters()]
        assert not any("layers.0.attn_res_mixer" in n for n in names)          # nothing to mix before the first layer
        assert any("layers.1.attn_res_mixer.proj_weight" in n for n in names) and \
            any("decoder.attn_res_head.norm_weight" in n for n in names)
        losses = tr.train()
        assert len(losses) == 3 and all(math.isfinite(x) for x in losses)
        biases = [m.router.expert_bias.clone() for m in tr.model.modules() if hasattr(m, "update_expert_bias")]
        assert biases and all(float(b.abs().max()) > 0 and abs(float(b.mean())) < 1e-6 for b in biases)
        tr.tcfg.save = str(tmp_path)
        tr.save_checkpoint()
        tr2 = make(5)
        assert tr2.load_checkpoint(str(tmp_path)) == 3
        for (n, a), (_, b) in zip(tr.model.state_dict().items(), tr2.model.state_dict().items()):
            assert torch.equal(a, b), n
        # full recompute replays the layers with the checkpoints travelling in the residual slot: same losses
        again = make(3, recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2).train()
        assert all(abs(a - b) < 1e-5 for a, b in zip(losses, again)), (losses, again)
    finally:
        ps.destroy_model_parallel()


def test_presets_resolve():
    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig

    c = TransformerConfig.from_dict(load_preset("kimi_k3.yaml", "models", "primus_b200"))
    kinds = [k for k, _ in c.layer_kinds]
    assert kinds.count("kda") == 69 and kinds.count("attention") == 24 and c.multi_latent_attention and c.mla_use_nope
    assert sum(c.moe_layer_pattern) == 92 and c.routed_expert_hidden_size == 3584
    c8 = TransformerConfig.from_dict(load_preset("kimi_k3_8L_official.yaml", "models", "primus_b200"))
    assert [k for k, _ in c8.layer_kinds] == ["kda"] * 3 + ["attention"] + ["kda"] * 3 + ["attention"]


def test_delta_attention_stack_of_the_hybrid_presets():
    """``linear_attention_type: kda`` in a Mamba-style stack: mixer layers alternate with MLP layers, key heads narrower than
    value heads, output gate and forget gate through bottlenecks, unbounded softplus decay."""
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(9)
    cfg = TransformerConfig(model_type="mamba", is_hybrid_model=True, linear_attention_type="kda", num_layers=4,
                            hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=256, params_dtype="fp32",
                            linear_num_key_heads=4, linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=16,
                            kda_use_full_rank_gate=False, kda_gate_lower_bound=None, kda_chunk_size=16)
    assert cfg.layer_kinds == [("kda", False), (None, True)] * 2
    m = GPTModel(cfg)
    assert sum(p.numel() for p in m.parameters()) == cfg.num_parameters()
    mixer = m.decoder.layers["0"].mixer
    assert mixer.f_b_proj.weight.shape == (32, 16) and mixer.g_b_proj.weight.shape == (64, 16)
    tok = torch.randint(0, 256, (2, 40))
    loss = m(tok, tok, None).mean()
    loss.backward()
    assert math.isfinite(float(loss)) and all(p.grad is not None for p in m.parameters())
    ps.destroy_model_parallel()


def test_multi_token_prediction_layer_has_no_attention_residuals():
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(12)
    m = GPTModel(_k3_cfg(mtp_num_layers=1))
    inner = m.mtp.layers[0].transformer_layer
    assert not inner.attn_res and not hasattr(inner, "mlp_res_mixer") and m.decoder.layers["5"].attn_res
    tok = torch.randint(0, 256, (2, 64))
    loss = m(tok, tok, torch.full((2, 64), 1.0 / 128))
    loss.backward()
    assert math.isfinite(float(loss)) and all(p.grad is not None for n, p in m.named_parameters() if n.startswith("mtp."))
    ps.destroy_model_parallel()
