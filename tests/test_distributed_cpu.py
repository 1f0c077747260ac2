"""Multi-process CPU (gloo) plumbing: DP with the distributed optimizer, TP (+SP), PP schedules and EP must
reproduce the single-process loss trajectory from identical initial weights and the same global batches."""
import dataclasses
import json

import pytest
import torch

from tests import dist_workers as W
from tests.mp_utils import run_ranks


def _single(kwargs):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps

    mc, tc = W.tiny_cfgs(**{**kwargs, "tp": 1, "pp": 1, "ep": 1, "cp": 1, "sp": False, "vpp": None, "schedule": "1f1b"})
    mck = _mc_kwargs(mc)
    full = W.full_reference_state(mck)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    W.load_from_full(tr, full)
    norms = []
    out = tr.train(on_step=lambda t, lv: norms.append(float(t.optimizer.grad_norm.item())))
    ps.destroy_model_parallel()
    _single.last_norms = norms
    return out, mck


def _mc_kwargs(mc):
    d = {f.name: getattr(mc, f.name) for f in dataclasses.fields(mc)}
    return d


CASES = {
    "dp2": dict(world=2, kw=dict()),
    "dp2_fsdp2": dict(world=2, kw=dict(fsdp=True)),
    # hybrid sharding: two groups of two ranks, sharded inside a group, replicated across
    "dp4_hsdp": dict(world=4, kw=dict(fsdp=True, extra_tc=dict(data_parallel_replicate_degree=2))),
    "dp2_bf16_grad_reduce": dict(world=2, kw=dict(extra_tc=dict(grad_reduce_in_bf16=True, overlap_grad_reduce=True))),
    "dp2_odc": dict(world=2, kw=dict(extra_tc=dict(enable_odc=True, overlap_grad_reduce=True))),
    "dp2_overlap_param_gather": dict(world=2, kw=dict(extra_tc=dict(overlap_param_gather=True, overlap_grad_reduce=True))),
    "dp2_pp2_overlap_param_gather": dict(world=4, kw=dict(pp=2, extra_tc=dict(overlap_param_gather=True))),
    "tp2_sp": dict(world=2, kw=dict(tp=2, sp=True)),
    "tp2_nosp": dict(world=2, kw=dict(tp=2, sp=False)),
    "tp2_sp_mla": dict(world=2, kw=dict(tp=2, sp=True, mla=True)),
    "tp2_nosp_mla": dict(world=2, kw=dict(tp=2, sp=False, mla=True)),
    "tp2_pp2_ep2_mla_moe": dict(world=8, kw=dict(tp=2, pp=2, ep=2, sp=True, mla=True, moe=True)),
    # head-split gated-delta-net / Kimi-delta-attention mixers (fused projections re-tiled block by block)
    "tp2_sp_qwen3_5": dict(world=2, kw=dict(tp=2, sp=True, layers=4, extra_mc=dict(
        experimental_attention_variant="gated_delta_net", linear_attention_freq=2, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_chunk_size=16,
        attention_output_gate=True, apply_layernorm_1p=True, rotary_percent=0.5, qk_layernorm=True))),
    "tp2_sp_pp2_kimi_k3": dict(world=4, kw=dict(tp=2, sp=True, pp=2, layers=6, extra_mc=dict(
        model_type="kimi_k3", q_lora_rank=32, kv_lora_rank=24, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16,
        mla_use_output_gate=True, linear_attention_freq="([1]*2+[0])*2", linear_num_key_heads=4, linear_num_value_heads=4,
        linear_key_head_dim=16, linear_value_head_dim=16, kda_chunk_size=16, attn_res_block_size=2, num_experts=4,
        moe_router_topk=2, moe_ffn_hidden_size=32, moe_layer_freq="([0]*1+[1]*5)", moe_shared_expert_intermediate_size=32,
        routed_expert_hidden_size=32, moe_router_score_function="sigmoid", gated_activation="situ"))),
    "tp2_sp_kda_hybrid": dict(world=2, kw=dict(tp=2, sp=True, layers=4, extra_mc=dict(
        model_type="mamba", is_hybrid_model=True, linear_attention_type="kda", linear_num_key_heads=4,
        linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=16, kda_use_full_rank_gate=False,
        kda_gate_lower_bound=None, kda_chunk_size=16))),
    # LFM2: channel-split gated short convolutions (with biases) between grouped-query attention layers
    "tp2_sp_lfm2": dict(world=2, kw=dict(tp=2, sp=True, layers=4, extra_mc=dict(
        lfm_layer_types=["conv", "full_attention", "conv", "conv"], conv_L_cache=3, conv_bias=True, qk_layernorm=True))),
    "tp2_sp_mamba_hybrid": dict(world=2, kw=dict(tp=2, sp=True, layers=6, extra_mc=dict(
        model_type="mamba", is_hybrid_model=True, hybrid_attention_ratio=0.34, mamba_state_dim=16, mamba_head_dim=16,
        mamba_num_groups=2, mamba_chunk_size=16))),
    "tp2_sp_pp2_deepseek_v4": dict(world=4, kw=dict(tp=2, sp=True, pp=2, layers=4, seq=128, extra_mc=dict(
        model_type="deepseek_v4", num_query_groups=1, kv_channels=32, qk_pos_emb_head_dim=8, q_lora_rank=32, o_lora_rank=16,
        o_groups=2, hc_mult=3, hc_sinkhorn_iters=6, compress_ratios="[0, 4, 128, 4]", compress_rope_theta=40000.0,
        index_topk=4, index_head_dim=16, index_n_heads=2, attn_sliding_window=8, num_experts=4, moe_router_topk=2,
        moe_ffn_hidden_size=32, moe_layer_freq=1, moe_shared_expert_intermediate_size=32,
        moe_router_score_function="sqrtsoftplus", activation_func_clamp_value=10.0, v4_indexer_distill_loss_coeff=0.1,
        num_hash_layers=3))),
    "dp2_tp2_replica_check": dict(world=4, kw=dict(tp=2, sp=True, extra_tc=dict(
        check_weight_hash_across_dp_replicas_interval=1, log_params_norm=True))),
    "pp2_1f1b": dict(world=2, kw=dict(pp=2)),
    "dp2_pp2_tp_pp_dp_mapping": dict(world=4, kw=dict(pp=2, extra_tc=dict(use_tp_pp_dp_mapping=True))),
    "tp2_pp2_ep2_tp_pp_dp_mapping": dict(world=8, kw=dict(tp=2, pp=2, ep=2, sp=True, moe=True,
                                                          extra_tc=dict(use_tp_pp_dp_mapping=True))),
    "pp2_interleaved": dict(world=2, kw=dict(pp=2, vpp=2, schedule="interleaved")),
    "pp2_warmup": dict(world=2, kw=dict(pp=2, vpp=2, schedule="interleaved", pp_warmup=True)),
    # uneven stages: a short last stage, a layout string, the embedding counted as a layer, interleaved chunks of 2-1-1-1
    "pp2_uneven_last": dict(world=2, kw=dict(pp=2, extra_tc=dict(decoder_last_pipeline_num_layers=1))),
    "pp2_layout_string": dict(world=2, kw=dict(pp=2, extra_tc=dict(pipeline_model_parallel_layout="Et|tttL"))),
    "pp2_account_embedding": dict(world=2, kw=dict(pp=2, layers=5, extra_tc=dict(account_for_embedding_in_pipeline_split=True))),
    "pp2_interleaved_uneven": dict(world=2, kw=dict(pp=2, vpp=2, layers=5, schedule="interleaved",
                                                    extra_tc=dict(decoder_first_pipeline_num_layers=2))),
    "pp2_zerobubble": dict(world=2, kw=dict(pp=2, schedule="zerobubble")),
    "pp2_zbv": dict(world=2, kw=dict(pp=2, schedule="zbv")),
    "pp2_zerobubble_manual_costs": dict(world=2, kw=dict(pp=2, schedule="zerobubble", extra_tc=dict(
        pp_cost_f=[1000, 1400], pp_cost_b=1200, pp_cost_w=700, pp_max_mem=4, debug_scheduler_table=True))),
    # every micro-batch travels through the pipeline as two / four sequence chunks (attention over the kept K / V)
    "pp2_seq_splits2": dict(world=2, kw=dict(pp=2, extra_tc=dict(num_seq_splits=2))),
    "pp2_tp2_seq_splits4": dict(world=4, kw=dict(pp=2, tp=2, sp=True, extra_tc=dict(num_seq_splits=4))),
    # node times measured in iterations 1-2, cost-driven table from iteration 3 on: same losses
    "pp2_zerobubble_replanned": dict(world=2, kw=dict(pp=2, schedule="zerobubble", iters=4, extra_tc=dict(
        zero_bubble_pipeline_timers_start_iter=1, zero_bubble_pipeline_timers_end_iter=3))),
    "pp2_zbv_replanned": dict(world=2, kw=dict(pp=2, schedule="zbv", iters=4, extra_tc=dict(
        zero_bubble_pipeline_timers_start_iter=1, zero_bubble_pipeline_timers_end_iter=3,
        zero_bubble_max_pending_backward=4))),
    # optimistic optimizer step validated after the cross-stage norm reduction; clip 1e-3 forces the redo path
    "pp2_zerobubble_post_validation": dict(world=2, kw=dict(pp=2, schedule="zerobubble",
                                                            extra_tc=dict(enable_optimizer_post_validation=True))),
    "pp2_zerobubble_post_validation_redo": dict(world=2, kw=dict(pp=2, schedule="zerobubble", clip=1e-3,
                                                                 extra_tc=dict(enable_optimizer_post_validation=True))),
    "pp2_post_validation_inverse": dict(world=2, kw=dict(pp=2, schedule="zerobubble", clip=1e-3, extra_tc=dict(
        enable_optimizer_post_validation=True, enable_exact_optimizer_post_validation=False))),
    "ep2_moe": dict(world=2, kw=dict(ep=2, moe=True)),
    # MoE layers under tensor + sequence parallelism: every rank routes its own sequence shard; without the
    # load-balancing loss, which is then a per-shard quantity, the trajectory is that of the single process
    "tp2_moe": dict(world=2, kw=dict(tp=2, sp=True, moe=True, extra_mc=dict(moe_aux_loss_coeff=0.0))),
    "tp2_ep2_moe": dict(world=4, kw=dict(tp=2, sp=True, ep=2, moe=True, extra_mc=dict(moe_aux_loss_coeff=0.0))),
    "tp2_ep2_moe_shared": dict(world=4, kw=dict(tp=2, sp=True, ep=2, moe=True, extra_mc=dict(
        moe_aux_loss_coeff=0.0, moe_shared_expert_intermediate_size=32))),
    "tp2_pp2": dict(world=4, kw=dict(tp=2, pp=2, sp=True)),
    "tp2_qkv_bias": dict(world=2, kw=dict(tp=2, sp=True, extra_mc=dict(add_qkv_bias=True))),
    "cp2": dict(world=2, kw=dict(cp=2)),
    "cp2_pp2": dict(world=4, kw=dict(cp=2, pp=2)),
    "cp2_allgather": dict(world=2, kw=dict(cp=2, cp_comm="allgather")),
    "cp2_allgather_mla": dict(world=2, kw=dict(cp=2, cp_comm="allgather", mla=True)),
    "cp2_ring": dict(world=2, kw=dict(cp=2, cp_comm="p2p")),
    "cp4_ring_mla": dict(world=4, kw=dict(cp=4, cp_comm="p2p", mla=True, seq=64)),
    "pp2_tied_embeddings": dict(world=2, kw=dict(pp=2, tied=True)),
    "pp2_interleaved_tied": dict(world=2, kw=dict(pp=2, vpp=2, schedule="interleaved", tied=True)),
    "tp2_sp_mtp": dict(world=2, kw=dict(tp=2, sp=True, mtp=1)),
    "tp2_nosp_mtp": dict(world=2, kw=dict(tp=2, sp=False, mtp=1)),
    "pp2_dp2_mtp": dict(world=4, kw=dict(pp=2, mtp=1)),
    "cp4_a2a_p2p": dict(world=4, kw=dict(cp=4, cp_comm="a2a+p2p", cp_sizes=[2, 2], seq=64)),
    # Kimi-K3: the running stream and the attention-residual checkpoints cross the stage boundary as one tensor
    "pp2_kimi_k3": dict(world=2, kw=dict(pp=2, layers=6, extra_mc=dict(
        model_type="kimi_k3", q_lora_rank=32, kv_lora_rank=24, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16,
        mla_use_output_gate=True, linear_attention_freq="([1]*2+[0])*2", linear_num_key_heads=4, linear_num_value_heads=4,
        linear_key_head_dim=16, linear_value_head_dim=16, kda_chunk_size=16, attn_res_block_size=2, num_experts=4,
        moe_router_topk=2, moe_ffn_hidden_size=32, moe_layer_freq="([0]*1+[1]*5)", moe_shared_expert_intermediate_size=32,
        routed_expert_hidden_size=32, moe_router_score_function="sigmoid", gated_activation="situ"))),
    # DeepSeek-V4: the hyper-connection streams cross the stage boundary; hash-routed layers on both stages
    "pp2_deepseek_v4": dict(world=2, kw=dict(pp=2, layers=4, seq=128, mtp=1, extra_mc=dict(
        model_type="deepseek_v4", num_query_groups=1, kv_channels=32, qk_pos_emb_head_dim=8, q_lora_rank=32, o_lora_rank=16,
        o_groups=2, hc_mult=3, hc_sinkhorn_iters=6, compress_ratios="[0, 4, 128, 4, 0]", compress_rope_theta=40000.0,
        index_topk=4, index_head_dim=16, index_n_heads=2, attn_sliding_window=8, num_experts=4, moe_router_topk=2,
        moe_ffn_hidden_size=32, moe_layer_freq=1, moe_shared_expert_intermediate_size=32,
        moe_router_score_function="sqrtsoftplus", num_hash_layers=3, activation_func_clamp_value=10.0))),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_parallel_matches_single_process(name, tmp_path):
    case = CASES[name]
    kw = dict(seq=32, gbs=8, mbs=2, iters=3, layers=4)
    kw.update(case["kw"])
    ref, mck = _single(kw)
    out = tmp_path / "losses.json"
    run_ranks(W.train_worker, case["world"], "gloo", args=(kw, mck, str(out)), timeout=240)
    got = json.loads(out.read_text())
    assert len(got) == len(ref)
    for a, b in zip(got, ref):
        assert abs(a - b) <= 2e-3 * max(1.0, abs(b)), f"{name}: {got} vs {ref}"


NORM_CASES = {
    # norm weights (and, without sequence parallelism, nothing else) are replicated over the tensor-parallel ranks
    "tp2_sp": dict(world=2, kw=dict(tp=2, sp=True)),
    "tp2_nosp": dict(world=2, kw=dict(tp=2, sp=False)),
    "tp2_pp2": dict(world=4, kw=dict(tp=2, pp=2, sp=True)),
    # multi-latent attention: the down-projections are replicated as well
    "tp2_sp_mla": dict(world=2, kw=dict(tp=2, sp=True, mla=True)),
    "tp2_nosp_mla": dict(world=2, kw=dict(tp=2, sp=False, mla=True)),
    "tp2_sp_kda_hybrid": dict(world=2, kw=dict(tp=2, sp=True, layers=4, extra_mc=dict(
        model_type="mamba", is_hybrid_model=True, linear_attention_type="kda", linear_num_key_heads=4,
        linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=16, kda_use_full_rank_gate=False,
        kda_gate_lower_bound=None, kda_chunk_size=16))),
    # whole-parameter optimizers: every expert-parallel rank owns different experts
    "ep2_moe_sgd": dict(world=2, kw=dict(ep=2, moe=True, opt="sgd", distopt=False)),
    "ep2_moe_adam": dict(world=2, kw=dict(ep=2, moe=True)),
    "tp2_ep2_moe": dict(world=4, kw=dict(tp=2, sp=True, ep=2, moe=True, extra_mc=dict(moe_aux_loss_coeff=0.0))),
}


@pytest.mark.parametrize("name", sorted(NORM_CASES))
def test_grad_norm_matches_single_process(name, tmp_path):
    """The global gradient norm (and so the clip coefficient) must not depend on the parallel layout: tensor-parallel
    duplicates are counted once, expert shards of all expert-parallel ranks are included."""
    case = NORM_CASES[name]
    kw = dict(seq=32, gbs=8, mbs=2, iters=2, layers=4, lr=1e-3)
    kw.update(case["kw"])
    ref, mck = _single(kw)
    ref_norms = list(_single.last_norms)
    out = tmp_path / "losses.json"
    run_ranks(W.train_worker, case["world"], "gloo", args=(kw, mck, str(out)), timeout=240)
    got = json.loads((tmp_path / "losses.json.norms").read_text())
    assert len(got) == len(ref_norms) and all(n > 0 for n in ref_norms)
    for a, b in zip(got, ref_norms):
        assert abs(a - b) <= 2e-3 * b, f"{name}: grad norms {got} vs {ref_norms}"


def test_evaluation_under_pipeline_parallelism(tmp_path):
    """The forward-only pipeline pass gives the validation loss of the single-process model."""
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps

    kw = dict(seq=32, gbs=8, mbs=2, iters=2, layers=4, extra_tc=dict(eval_iters=2))
    ref, mck = _single(kw)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(**kw)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    W.load_from_full(tr, W.full_reference_state(mck))
    tr.train()
    want = tr.evaluate(2)
    ps.destroy_model_parallel()
    for name, extra in (("pp2", dict(pp=2)), ("pp2i", dict(pp=2, vpp=2, schedule="interleaved"))):
        out = tmp_path / f"{name}.json"
        run_ranks(W.train_worker, 2, "gloo", args=({**kw, **extra}, mck, str(out)), timeout=240)
        got = json.loads((tmp_path / f"{name}.json.eval").read_text())
        assert abs(got - want) <= 2e-3 * max(1.0, abs(want)), (name, got, want)
