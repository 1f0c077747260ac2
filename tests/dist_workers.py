"""Rank functions for the multi-process CPU (gloo) tests; importable by spawned children."""
import torch


def tiny_cfgs(tp=1, pp=1, ep=1, cp=1, sp=False, moe=False, seq=64, gbs=8, mbs=2, iters=4, schedule="1f1b", vpp=None, layers=4,
              pp_warmup=False, cp_comm="a2a", mla=False, fsdp=False, cp_sizes=None, tied=False, mtp=0, opt="adam",
              distopt=True, hidden=64, heads=4, ffn=128, vocab=512, lr=1e-2, clip=1.0, recompute=None, extra_mc=None,
              extra_tc=None):
    from primus_b200.engine.trainer import TrainConfig
    from primus_b200.models.config import TransformerConfig

    kw = dict(num_layers=layers, hidden_size=hidden, ffn_hidden_size=ffn, num_attention_heads=heads, num_query_groups=2,
              vocab_size=vocab, params_dtype="fp32", tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
              expert_model_parallel_size=ep, context_parallel_size=cp, sequence_parallel=sp, make_vocab_size_divisible_by=64,
              virtual_pipeline_model_parallel_size=vpp, cp_comm_type=cp_comm,
              hierarchical_context_parallel_sizes=cp_sizes, untie_embeddings_and_output_weights=not tied,
              mtp_num_layers=mtp)
    if mla:
        kw.update(multi_latent_attention=True, kv_lora_rank=32, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16)
    if moe:
        kw.update(num_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_layer_freq=[0, 1] * (layers // 2),
                  moe_aux_loss_coeff=1e-2)
    if recompute:
        kw.update(recompute)
    if extra_mc:
        kw.update(extra_mc)
    mc = TransformerConfig(**kw)
    tc = TrainConfig(micro_batch_size=mbs, global_batch_size=gbs, seq_length=seq, train_iters=iters, lr=lr,
                     lr_decay_style="constant", weight_decay=0.01, clip_grad=clip, pipeline_schedule=schedule,
                     log_interval=1, pp_warmup=pp_warmup, use_torch_fsdp2=fsdp, optimizer=opt,
                     use_distributed_optimizer=distopt, **(extra_tc or {}))
    return mc, tc


def full_reference_state(mc_kwargs, seed=7):
    """State dict of the un-sharded single-process model (deterministic)."""
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    kw = dict(mc_kwargs)
    kw.update(tensor_model_parallel_size=1, pipeline_model_parallel_size=1, expert_model_parallel_size=1,
              context_parallel_size=1,
              sequence_parallel=False, virtual_pipeline_model_parallel_size=None)
    torch.manual_seed(seed)
    m = GPTModel(TransformerConfig(**kw), "cpu")
    return {k: v.detach().clone() for k, v in m.state_dict().items()}


def load_from_full(trainer, full_sd):
    """Copy the matching slice of the full model into every parameter of this rank's chunks."""
    from primus_b200.engine import checkpoint as C

    st, cfg = trainer.st, trainer.mcfg
    for m in trainer.model_chunks:
        for name, p in m.named_parameters():
            full = full_sd[name]
            spec = C.shard_spec(name, p, cfg, st)
            if spec["kind"] == "qkv":
                # full tensor is [q | k | v]; shard every part separately
                hq, hkv, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.kv_channels
                q, k, v = full[:hq * d], full[hq * d:(hq + hkv) * d], full[(hq + hkv) * d:]
                n, i = spec["count"], spec["index"]
                part = torch.cat([t.chunk(n, 0)[i] for t in (q, k, v)], 0)
            else:
                part = C.slice_global(name, full, spec)
            if hasattr(p, "device_mesh"):      # fully sharded parameter: hand every rank its shard of the full tensor
                from torch.distributed.tensor import distribute_tensor

                p.data.copy_(distribute_tensor(part.to(p.dtype), p.device_mesh, p.placements))
            else:
                p.data.copy_(part)
    C._refresh_master_weights(trainer)


def train_worker(rank, world, kwargs, mc_kwargs_full, outq_path):
    import json

    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps

    full_sd = full_reference_state(mc_kwargs_full)
    ps.destroy_model_parallel()
    mc, tc = tiny_cfgs(**kwargs)
    ps.initialize_model_parallel(tp=mc.tensor_model_parallel_size, pp=mc.pipeline_model_parallel_size,
                                 ep=mc.expert_model_parallel_size, cp=mc.context_parallel_size, virtual_pp=mc.virtual_pipeline_model_parallel_size,
                                 hierarchical_cp_sizes=mc.hierarchical_context_parallel_sizes,
                                 tp_pp_dp_mapping=tc.use_tp_pp_dp_mapping)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    load_from_full(tr, full_sd)
    norms = []
    losses = tr.train(on_step=lambda t, lv: norms.append(float(t.optimizer.grad_norm.item())))
    if (kwargs.get("extra_tc") or {}).get("zero_bubble_pipeline_timers_end_iter"):
        rep = tr.pp_replan_report          # the cost-driven table was built and installed for the later iterations
        assert rep is not None and rep["makespan"] <= rep["fixed_makespan"] + 1e-9, rep
        key = (tc.pipeline_schedule, ps.get_state().pp, len(losses) and tr.num_microbatches, ps.get_state().virtual_pp)
        assert tr._pp_schedule_cache[key] is rep
    if kwargs.get("extra_tc", {}) and kwargs["extra_tc"].get("eval_iters"):
        val = tr.evaluate(kwargs["extra_tc"]["eval_iters"])
        if rank == 0:
            with open(outq_path + ".eval", "w") as f:
                json.dump(val, f)
    if rank == 0:
        with open(outq_path, "w") as f:
            json.dump(losses, f)
        with open(outq_path + ".norms", "w") as f:
            json.dump(norms, f)
