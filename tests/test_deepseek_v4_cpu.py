"""DeepSeek-V4 building blocks against direct statements of their definitions: hyper-connections, the compressor, the
indexer, the joint local + compressed attention with a sink, the rotary / inverse-rotary pair, the hash router, and the
whole stack through the trainer.  (The reference keeps eager oracles of the same operations in
primus/backends/megatron/core/transformer/v4_attention_kernels/_eager/reference.py and tests them in
tests/unit_tests/megatron/transformer/deepseek_v4/.)"""
import math

import pytest
import torch

from primus_b200.models import deepseek_v4 as V


def test_sinkhorn_and_hyper_connections():
    torch.manual_seed(0)
    m = V.sinkhorn(torch.rand(5, 4, 4) + 0.01, 30)
    assert torch.allclose(m.sum(-1), torch.ones(5, 4), atol=1e-3) and torch.allclose(m.sum(-2), torch.ones(5, 4), atol=1e-4)
    K, D, T = 3, 16, 7
    mix = V.HyperMixer(D, K, 1e-6, 20, "cpu")
    x = torch.randn(T, K, D)
    pre, post, comb = mix.weights(x)
    assert pre.shape == (T, K) and comb.shape == (T, K, K) and (pre > 0).all() and (post > 0).all() and (post < 2).all()
    seen = {}

    def sub(h):
        seen["h"] = h
        return torch.tanh(h)

    out = mix.apply(x, sub)
    assert torch.allclose(seen["h"], (pre[..., None] * x).sum(1), atol=1e-6)
    ref = post[..., None] * torch.tanh(seen["h"])[:, None] + torch.einsum("thk,tkd->thd", comb, x)
    assert torch.allclose(out, ref, atol=1e-6)
    # zero projection, zero offsets: every stream is read with weight 1/2, written with weight 1, streams mix evenly
    with torch.no_grad():
        mix.fn.weight.zero_()
    pre, post, comb = mix.weights(x)
    assert torch.allclose(pre, torch.full((T, K), 0.5 + 1e-6)) and torch.allclose(post, torch.ones(T, K))
    assert torch.allclose(comb, torch.full((T, K, K), 1.0 / K), atol=1e-4)
    head = V.HyperHead(D, K, 1e-6, "cpu")
    with torch.no_grad():
        head.fn.weight.zero_()
    assert torch.allclose(head(x), 0.5 * x.sum(1), atol=1e-4)


@pytest.mark.parametrize("ratio", [4, 128])
def test_compressor_pools_windows(ratio):
    torch.manual_seed(1)
    B, S, H, d = 2, 2 * max(ratio, 8), 24, 8
    comp = V.Compressor(H, d, ratio, 1e-6, 0.2, torch.float32, "cpu")
    with torch.no_grad():
        comp.kv_norm.weight.uniform_(0.5, 1.5)
    x = torch.randn(B * S, H)
    out = comp(x, B)
    assert out.shape == (B, S // ratio, d)
    w = comp.wkv_gate.weight
    width = w.shape[0] // 2
    kv, sc = (x @ w[:width].t()).view(B, S, width), (x @ w[width:].t()).view(B, S, width)
    for b in range(B):
        for n in range(S // ratio):
            rows = slice(n * ratio, (n + 1) * ratio)
            if ratio == 4:      # this window through the first half of the channels, the previous through the second
                prev = slice((n - 1) * ratio, n * ratio)
                k_ = torch.cat([kv[b, rows, :d], kv[b, prev, d:] if n else torch.zeros(ratio, d)])
                s_ = torch.cat([sc[b, rows, :d], sc[b, prev, d:] if n else torch.zeros(ratio, d)])
            else:
                k_, s_ = kv[b, rows], sc[b, rows]
            pooled = (k_ * torch.softmax(s_ + comp.ape, 0)).sum(0)
            pooled = pooled * torch.rsqrt(pooled.pow(2).mean() + 1e-6) * comp.kv_norm.weight
            assert torch.allclose(out[b, n], pooled, atol=1e-5), (b, n)


def test_window_mask_and_rotary_pair():
    m = V.window_mask(12, 3, 4, "cpu")
    assert m[:, 0].tolist() == [False] * 3 + [True] * 9 and m[:, 2].tolist() == [False] * 11 + [True]
    torch.manual_seed(2)
    inv = V.yarn_inv_freq(8, 10000.0)
    x = torch.randn(2, 5, 3, 16)
    pos = torch.arange(5)[None].expand(2, 5)
    y = V.rope_interleaved(x, pos, inv, 8)
    assert torch.equal(y[..., :8], x[..., :8])                                  # only the last channels turn
    assert torch.allclose(V.rope_interleaved(y, pos, inv, 8, inverse=True), x, atol=1e-6)
    a, b = x[0, 3, 0, 8], x[0, 3, 0, 9]                                          # pair (0, 1) of the rotary part
    ang = 3 * inv[0]
    assert torch.allclose(y[0, 3, 0, 8], a * torch.cos(ang) - b * torch.sin(ang), atol=1e-6)
    # long wavelengths are stretched by the factor, short ones kept
    base, yarn = V.yarn_inv_freq(64, 40000.0), V.yarn_inv_freq(64, 40000.0, 4.0, 32.0, 1.0, 65536)
    assert torch.allclose(yarn[0], base[0]) and torch.allclose(yarn[-1], base[-1] / 4.0)


def _naive_joint(q, kv, sink, window, scale, pool=None, pool_mask=None, gathered=None, ok=None):
    B, H, S, D = q.shape
    out = torch.zeros(B, H, S, D)
    for b in range(B):
        for h in range(H):
            for t in range(S):
                lo = 0 if not window else max(0, t - window + 1)
                keys = [kv[b, j] for j in range(lo, t + 1)]
                if pool is not None:
                    keys += [pool[b, p] for p in range(pool.shape[1]) if pool_mask[t, p]]
                if gathered is not None:
                    keys += [gathered[b, t, k] for k in range(gathered.shape[2]) if ok[b, t, k]]
                Kt = torch.stack(keys)
                logits = (Kt @ q[b, h, t]) * scale
                if sink is not None:
                    logits = torch.cat([logits, sink[h:h + 1]])
                p = torch.softmax(logits, 0)[: len(keys)]
                out[b, h, t] = p @ Kt
    return out


def test_joint_attention_matches_a_per_query_loop():
    torch.manual_seed(3)
    B, H, S, D, P, K = 2, 3, 16, 8, 4, 3
    q, kv = torch.randn(B, H, S, D), torch.randn(B, S, D)
    sink = torch.randn(H)
    scale = D ** -0.5
    assert torch.allclose(V.joint_attention(q, kv, sink, 5, scale), _naive_joint(q, kv, sink, 5, scale), atol=1e-5)
    assert torch.allclose(V.joint_attention(q, kv, None, 0, scale), _naive_joint(q, kv, None, 0, scale), atol=1e-5)
    pool, mask = torch.randn(B, P, D), V.window_mask(S, P, 4, "cpu")
    assert torch.allclose(V.joint_attention(q, kv, sink, 5, scale, pool=pool, pool_mask=mask),
                          _naive_joint(q, kv, sink, 5, scale, pool=pool, pool_mask=mask), atol=1e-5)
    gathered, ok = torch.randn(B, S, K, D), torch.rand(B, S, K) > 0.4
    out, probs = V.joint_attention(q, kv, sink, 5, scale, gathered=gathered, gathered_ok=ok, return_gathered_probs=True)
    assert torch.allclose(out, _naive_joint(q, kv, sink, 5, scale, gathered=gathered, ok=ok), atol=1e-5)
    assert probs.shape == (B, H, S, K) and float(probs.masked_select(~ok[:, None].expand_as(probs)).abs().max()) == 0.0
    # a very large sink logit takes (almost) all the probability: the output vanishes
    assert V.joint_attention(q, kv, torch.full((H,), 40.0), 5, scale).abs().max() < 1e-10


def _v4_cfg(**over):
    from primus_b200.models.config import TransformerConfig

    kw = dict(model_type="deepseek_v4", num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4,
              num_query_groups=1, kv_channels=32, qk_pos_emb_head_dim=8, vocab_size=256, params_dtype="fp32",
              q_lora_rank=32, o_lora_rank=16, o_groups=2, hc_mult=3, hc_sinkhorn_iters=6,
              compress_ratios="[0, 4, 128, 4]", compress_rope_theta=40000.0, rotary_scaling_factor=4.0,
              original_max_position_embeddings=64, index_topk=4, index_head_dim=16, index_n_heads=2,
              attn_sliding_window=8, num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=32, moe_layer_freq=1,
              moe_shared_expert_intermediate_size=32, moe_router_score_function="sqrtsoftplus",
              moe_router_enable_expert_bias=True, moe_router_topk_scaling_factor=1.5, num_hash_layers=2,
              activation_func_clamp_value=10.0, untie_embeddings_and_output_weights=True)
    kw.update(over)
    return TransformerConfig(**kw)


def test_indexer_picks_finished_windows_only():
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(4)
    cfg = _v4_cfg(index_topk=3)
    att = V.V4Attention(cfg, 1, "cpu", 1)
    B, S = 2, 32
    y = torch.randn(B * S, 64)
    pos = torch.arange(S).repeat(B).view(B, S)
    idx, scores = att.indexer(y, pos, B)
    assert idx.shape == (B, S, 3)
    for t in range(S):
        visible = (t + 1) // 4                       # windows [4 s, 4 s + 4) that have ended by token t
        picked = idx[:, t][idx[:, t] >= 0]
        assert (picked < visible).all() and (idx[:, t] >= 0).sum(-1).eq(min(3, visible)).all()
    assert torch.isneginf(scores[idx < 0]).all()
    ps.destroy_model_parallel()


@pytest.mark.parametrize("layer", [0, 1, 2])
def test_attention_sees_relative_positions_only(layer):
    """Keys and values share one rotated latent and the output is rotated back by the query position: moving the whole
    sequence along the position axis (by a multiple of the compression ratio, so that the pooled entries move with it)
    leaves the layer's output unchanged."""
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(5)
    # no stretching of long wavelengths here: the pooled entries are rotated at ``s * ratio`` whatever the offset
    att = V.V4Attention(_v4_cfg(compress_ratios="[0, 0, 0, 0]"), layer, "cpu", 1)
    x = torch.randn(2 * 32, 64)
    base = torch.arange(32, dtype=torch.int32).repeat(2)
    a = att(x, None, (None, None, base, None), 2)[0]
    b = att(x, None, (None, None, base + 1000, None), 2)[0]
    assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()
    ps.destroy_model_parallel()


def test_sqrtsoftplus_and_hash_routing():
    from primus_b200.ops import moe as moe_ops

    torch.manual_seed(6)
    logits = torch.randn(10, 8)
    bias = torch.randn(8) * 0.1
    probs, idx, full = moe_ops.router_scores(logits, 2, "sqrtsoftplus", False, bias, 1.5)
    s = torch.sqrt(torch.nn.functional.softplus(logits))
    assert torch.allclose(full, s) and torch.equal(idx, (s + bias).topk(2, -1).indices)      # the bias only selects
    w = s.gather(1, idx)
    assert torch.allclose(probs, 1.5 * w / w.sum(-1, keepdim=True), atol=1e-6)
    table = V.hash_table(50, 8, 2, seed=3)
    assert table.shape == (50, 2) and (table[:, 0] != table[:, 1]).all() and torch.equal(table, V.hash_table(50, 8, 2, 3))
    tok = torch.randint(0, 50, (10,))
    probs, idx, _ = moe_ops.router_scores(logits, 2, "sqrtsoftplus", False, bias, 1.5, fixed_idx=table[tok])
    assert torch.equal(idx, table[tok].long())                                               # experts from the table ...
    w = s.gather(1, idx)
    assert torch.allclose(probs, 1.5 * w / w.sum(-1, keepdim=True), atol=1e-6)              # ... weights from the gate


def test_indexer_distillation_reaches_the_indexer_only():
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(7)
    tok = torch.randint(0, 256, (2, 128))
    grads = {}
    for coeff in (0.0, 0.5):
        torch.manual_seed(8)
        m = GPTModel(_v4_cfg(v4_indexer_distill_loss_coeff=coeff))
        m(tok, tok, None).mean().backward()
        grads[coeff] = {n: (None if p.grad is None else p.grad.clone()) for n, p in m.named_parameters()}
    idx_names = [n for n in grads[0.0] if ".indexer." in n]
    assert idx_names and all(grads[0.0][n] is None for n in idx_names)          # the top-k choice passes no gradient
    assert all(grads[0.5][n] is not None and float(grads[0.5][n].abs().max()) > 0 for n in idx_names)
    for n in grads[0.0]:
        if ".indexer." not in n:                                                # the rest of the model does not feel it
            assert torch.allclose(grads[0.0][n], grads[0.5][n], atol=1e-7), n
    ps.destroy_model_parallel()


def test_deepseek_v4_stack_trains_and_resumes(tmp_path):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    keys = ("model_type", "num_query_groups", "kv_channels", "qk_pos_emb_head_dim", "q_lora_rank", "o_lora_rank",
            "o_groups", "hc_mult", "hc_sinkhorn_iters", "compress_ratios", "compress_rope_theta", "rotary_scaling_factor",
            "original_max_position_embeddings", "index_topk", "index_head_dim", "index_n_heads", "attn_sliding_window",
            "num_experts", "moe_router_topk", "moe_ffn_hidden_size", "moe_layer_freq",
            "moe_shared_expert_intermediate_size", "moe_router_score_function", "moe_router_enable_expert_bias",
            "moe_router_topk_scaling_factor", "num_hash_layers", "activation_func_clamp_value")
    extra = {k: v for k, v in vars(_v4_cfg()).items() if k in keys}

    def make(iters, **more):
        mc, tc = W.tiny_cfgs(seq=128, gbs=4, mbs=2, iters=iters, layers=4, extra_mc=dict(extra, **more))
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        return Trainer(mc, tc, device="cpu", log_fn=lambda s: None)

    try:
        tr = make(3)
        names = dict(tr.model.named_parameters())
        assert "decoder.layers.1.self_attention.indexer.w_iuq.weight" in names and \
            "decoder.layers.2.self_attention.compressor.ape" in names and \
            "decoder.layers.0.self_attention.compressor.ape" not in names and "decoder.hc_head.base" in names
        assert hasattr(tr.model.decoder.layers["1"].mlp.router, "tid2eid") and \
            not hasattr(tr.model.decoder.layers["2"].mlp.router, "tid2eid")
        losses = tr.train()
        assert len(losses) == 3 and all(math.isfinite(x) for x in losses)
        tr.tcfg.save = str(tmp_path)
        tr.save_checkpoint()
        tr2 = make(5)
        with torch.no_grad():       # the hash table is state of the checkpoint, not of the seed
            tr2.model.decoder.layers["0"].mlp.router.tid2eid.zero_()
        assert tr2.load_checkpoint(str(tmp_path)) == 3
        for (n, a), (_, b) in zip(tr.model.state_dict().items(), tr2.model.state_dict().items()):
            assert torch.equal(a, b), n
        again = make(3, recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2).train()
        assert all(abs(a - b) < 1e-5 for a, b in zip(losses, again)), (losses, again)
    finally:
        ps.destroy_model_parallel()


def test_presets_resolve():
    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig

    flash = TransformerConfig.from_dict(load_preset("deepseek_v4_flash.yaml", "models", "primus_b200"))
    assert len(flash.compress_ratio_list) == 43 and flash.compress_ratio_list[:4] == [0, 0, 4, 128]
    assert 280e9 < flash.num_parameters() < 290e9
    pro = TransformerConfig.from_dict(load_preset("deepseek_v4_pro.yaml", "models", "primus_b200"))
    assert len(pro.compress_ratio_list) == 61 and pro.o_groups == 16 and pro.hc_mult == 4


def test_multi_token_prediction_with_hyper_connections():
    """Every depth copies its projected input into the streams, runs a layer of the family's kind (with the compression
    ratio listed behind the decoder layers) and collapses the streams with a head of its own."""
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(10)
    cfg = _v4_cfg(compress_ratios="[0, 4, 128, 4, 128]", mtp_num_layers=1)
    assert cfg.compress_ratio_list == [0, 4, 128, 4] and cfg.compress_ratio_mtp == [128]
    m = GPTModel(cfg)
    inner = m.mtp.layers[0].transformer_layer
    assert inner.self_attention.ratio == 128 and inner.hyper and hasattr(m.mtp.layers[0], "hc_head")
    tok = torch.randint(0, 256, (2, 128))
    w = torch.full((2, 128), 1.0 / 256)
    with_mtp = m(tok, tok, w)
    cfg0 = _v4_cfg(compress_ratios="[0, 4, 128, 4, 128]")
    torch.manual_seed(10)
    plain = GPTModel(cfg0)(tok, tok, w)
    assert float(with_mtp) > float(plain) > 0            # the depth adds its scaled loss on top of the same main loss
    with_mtp.backward()
    assert all(p.grad is not None for n, p in m.named_parameters() if n.startswith("mtp.") and ".indexer." not in n)
    ps.destroy_model_parallel()
