"""Weight conversion Hugging Face <-> engine: logits of the engine's model (plain PyTorch path, fp32, CPU) must match
the Hugging Face implementation of the same architecture with the same random weights."""
import pytest
import torch

from primus_b200.engine import hf_convert as H

transformers = pytest.importorskip("transformers")


def _engine_logits(hf_model, hf_cfg_dict, tokens, **extra):
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    kw = H.config_from_hf(hf_cfg_dict)
    kw.update(params_dtype="fp32", seq_length=tokens.shape[1], make_vocab_size_divisible_by=8, **extra)
    cfg = TransformerConfig(**kw)
    model = GPTModel(cfg, "cpu")
    sd = H.hf_to_internal({k: v.detach().clone() for k, v in hf_model.state_dict().items()}, cfg)
    missing = [k for k in model.state_dict() if k not in sd]
    assert not missing, missing
    model.load_state_dict(sd, strict=True)
    with torch.no_grad():
        logits = model(tokens)
    # round trip of the converter
    back = H.internal_to_hf(sd, cfg, stacked_experts=any(k.endswith('experts.gate_up_proj') for k in hf_model.state_dict()))
    for k, v in hf_model.state_dict().items():
        if k in back:
            assert torch.equal(back[k], v), k
    return logits[:, : cfg.vocab_size], cfg


def _check(hf_model, hf_cfg, tokens, tol=2e-4, **extra):
    hf_model.eval()
    with torch.no_grad():
        ref = hf_model(tokens).logits.reshape(-1, hf_cfg.vocab_size)
    got, _ = _engine_logits(hf_model, hf_cfg.to_dict(), tokens, **extra)
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), (err, ref.abs().max().item())


def test_llama_matches_hf():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    c = LlamaConfig(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=250, rope_theta=500000.0, rms_norm_eps=1e-5,
                    max_position_embeddings=128, tie_word_embeddings=False, attention_bias=False)
    _check(LlamaForCausalLM(c), c, torch.randint(0, 250, (2, 24)))


def test_qwen2_with_qkv_bias_matches_hf():
    Q = pytest.importorskip("transformers.models.qwen2")
    torch.manual_seed(5)
    c = Q.Qwen2Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=250, rope_theta=1e6, max_position_embeddings=128,
                      tie_word_embeddings=False, use_sliding_window=False)
    m = Q.Qwen2ForCausalLM(c)
    for n, p in m.named_parameters():
        if n.endswith(("q_proj.bias", "k_proj.bias", "v_proj.bias")):
            torch.nn.init.normal_(p, std=0.5)           # zero-initialised by default: make the biases matter
    _check(m, c, torch.randint(0, 250, (2, 24)))


def test_qwen3_dense_matches_hf():
    Q = pytest.importorskip("transformers.models.qwen3")
    torch.manual_seed(1)
    c = Q.Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, vocab_size=250, rope_theta=1e6, max_position_embeddings=128,
                      tie_word_embeddings=False)
    _check(Q.Qwen3ForCausalLM(c), c, torch.randint(0, 250, (1, 20)))


def test_qwen3_moe_matches_hf():
    Q = pytest.importorskip("transformers.models.qwen3_moe")
    torch.manual_seed(2)
    c = Q.Qwen3MoeConfig(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=250, num_experts=8,
                         num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                         max_position_embeddings=128, tie_word_embeddings=False, router_aux_loss_coef=0.0)
    _check(Q.Qwen3MoeForCausalLM(c), c, torch.randint(0, 250, (1, 16)))


def test_deepseek_v3_matches_hf():
    D = pytest.importorskip("transformers.models.deepseek_v3")
    torch.manual_seed(3)
    c = D.DeepseekV3Config(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1,
                           num_experts_per_tok=2, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16,
                           qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, n_group=2, topk_group=1,
                           routed_scaling_factor=2.5, norm_topk_prob=True, vocab_size=250, max_position_embeddings=128,
                           rope_scaling=None, tie_word_embeddings=False)
    m = D.DeepseekV3ForCausalLM(c)
    with torch.no_grad():  # make the selection bias matter
        for layer in m.model.layers[1:]:
            layer.mlp.gate.e_score_correction_bias.copy_(torch.randn(8) * 0.1)
            layer.mlp.gate.weight.copy_(torch.randn_like(layer.mlp.gate.weight) * 0.5)
    _check(m, c, torch.randint(0, 250, (1, 16)))


def test_mixtral_matches_hf():
    from transformers import MixtralConfig, MixtralForCausalLM

    torch.manual_seed(4)
    c = MixtralConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=250, num_local_experts=4, num_experts_per_tok=2,
                      max_position_embeddings=128, tie_word_embeddings=False, router_aux_loss_coef=0.0,
                      sliding_window=None)
    m = MixtralForCausalLM(c)
    _check(m, c, torch.randint(0, 250, (1, 16)))
    # the layout of published checkpoints (block_sparse_moe.experts.N.w1 / w3 / w2) converts to the same weights
    from primus_b200.models.config import TransformerConfig

    cfg = TransformerConfig(**H.config_from_hf(c.to_dict()), params_dtype="fp32", seq_length=16,
                            make_vocab_size_divisible_by=8)
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    new = H.hf_to_internal(sd, cfg)
    old = dict(sd)
    for L in range(2):
        h = f"model.layers.{L}."
        gu, dn = old.pop(h + "mlp.experts.gate_up_proj"), old.pop(h + "mlp.experts.down_proj")
        old[h + "block_sparse_moe.gate.weight"] = old.pop(h + "mlp.gate.weight")
        for e in range(4):
            old[h + f"block_sparse_moe.experts.{e}.w1.weight"] = gu[e, :96]
            old[h + f"block_sparse_moe.experts.{e}.w3.weight"] = gu[e, 96:]
            old[h + f"block_sparse_moe.experts.{e}.w2.weight"] = dn[e]
    conv = H.hf_to_internal(old, cfg)
    assert conv.keys() == new.keys() and all(torch.equal(conv[k], new[k]) for k in new)


def test_lfm2_moe_matches_hf():
    """Short convolutions + attention, two dense layers, then sigmoid-scored experts whose bias only steers the selection."""
    T = pytest.importorskip("transformers.models.lfm2_moe")

    torch.manual_seed(6)
    c = T.Lfm2MoeConfig(vocab_size=250, hidden_size=64, intermediate_size=128, moe_intermediate_size=48,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                        layer_types=["conv", "full_attention", "conv", "full_attention"], conv_L_cache=3, conv_bias=False,
                        num_dense_layers=1, num_experts=8, num_experts_per_tok=2, use_expert_bias=True,
                        norm_topk_prob=True, routed_scaling_factor=1.5, tie_word_embeddings=True)
    m = T.Lfm2MoeForCausalLM(c)
    with torch.no_grad():
        for layer in m.model.layers[1:]:
            layer.feed_forward.expert_bias.copy_(torch.randn(8) * 0.3)      # makes the selection differ from plain top-k
            layer.feed_forward.experts.gate_up_proj.normal_(0, 0.05)
            layer.feed_forward.experts.down_proj.normal_(0, 0.05)
    _check(m, c, torch.randint(0, 250, (2, 24)))
    kw = H.config_from_hf(c.to_dict())
    assert kw["moe_layer_freq"] == [0, 1, 1, 1] and kw["moe_router_score_function"] == "sigmoid"
    assert kw["moe_router_topk_scaling_factor"] == 1.5 and kw["moe_ffn_hidden_size"] == 48


def test_qwen3_5_moe_matches_hf():
    """Gated-delta-net layers with grouped key heads, gated full attention with partial rotary embedding, zero-centred norm
    gains and a gated shared expert."""
    Q = pytest.importorskip("transformers.models.qwen3_5_moe")
    torch.manual_seed(7)
    c = Q.Qwen3_5MoeTextConfig(vocab_size=256, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16,
                               linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                               moe_intermediate_size=32, shared_expert_intermediate_size=32, num_experts_per_tok=2,
                               num_experts=4, full_attention_interval=4, max_position_embeddings=256,
                               tie_word_embeddings=False)
    m = Q.Qwen3_5MoeForCausalLM(c)
    with torch.no_grad():       # the published initialisation leaves several tensors at zero / one: make every term count
        for n, p in m.named_parameters():
            if "norm" in n or "gate.weight" in n or "experts" in n or "dt_bias" in n:
                p.normal_(0.0, 0.1)
    try:
        _check(m, c, torch.randint(0, 256, (2, 96)), tol=5e-4, linear_chunk_size=32)
    finally:
        from primus_b200.ops import fused

        fused.set_zero_centered_gamma(False)


def test_train_from_hf_weights_export_and_offline_conversion(tmp_path):
    """``pretrained_hf_path`` -> a step of training -> ``export_hf_path``; the exported weights load into the Hugging Face
    model again, and the offline converter reads the engine checkpoint of the same run into the same tensors."""
    from safetensors.torch import load_file, save_file
    from transformers import LlamaConfig, LlamaForCausalLM

    from primus_b200.engine.pretrain import PretrainTrainer
    from primus_b200.parallel import state as ps
    from primus_b200.tools import convert_checkpoint

    torch.manual_seed(11)
    c = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, vocab_size=256, max_position_embeddings=128, tie_word_embeddings=False)
    hf = LlamaForCausalLM(c)
    src = tmp_path / "hf_in"
    src.mkdir()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(c.to_json_string())
    params = dict(H.config_from_hf(c.to_dict()), params_dtype="fp32", make_vocab_size_divisible_by=64, seq_length=32,
                  micro_batch_size=2, global_batch_size=2, train_iters=1, lr=0.0, weight_decay=0.0, mock_data=True,
                  log_interval=1, pretrained_hf_path=str(src), export_hf_path=str(tmp_path / "hf_out"),
                  save=str(tmp_path / "ckpt"), use_distributed_optimizer=True)
    ps.destroy_model_parallel()
    try:
        tr = PretrainTrainer.__new__(PretrainTrainer)
        tr.params, tr.runtime_state, tr.world_size, tr.local_rank = params, None, 1, 0
        tr.init()
        tok = torch.randint(0, 256, (1, 16))
        with torch.no_grad():
            assert torch.allclose(tr.engine.model(tok)[:, :256], hf(tok).logits.reshape(-1, 256), atol=2e-4)
        tr.train()
    finally:
        ps.destroy_model_parallel()
    out = load_file(str(tmp_path / "hf_out" / "model.safetensors"))
    for k, v in hf.state_dict().items():        # learning rate 0: the exported weights are the imported ones
        assert torch.equal(out[k], v), k
    assert convert_checkpoint.main(["engine-to-hf", "--load", str(tmp_path / "ckpt"), "--output", str(tmp_path / "hf2")]) == 0
    out2 = load_file(str(tmp_path / "hf2" / "model.safetensors"))
    assert all(torch.equal(out2[k], v) for k, v in hf.state_dict().items())
    assert convert_checkpoint.main(["hf-to-engine", "--hf", str(src), "--output", str(tmp_path / "full.pt"),
                                    "--params-dtype", "fp32"]) == 0
    full = torch.load(tmp_path / "full.pt", weights_only=False)
    assert set(full["state"]) == set(tr.engine.model.state_dict())
