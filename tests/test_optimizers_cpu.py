"""SGD / Muon update rules, evaluation loop and tokenizer builder (CPU)."""
import torch

from primus_b200.parallel import matrix_optimizers as MO


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in ((64, 32), (32, 96), (48, 48)):
        m = torch.randn(*shape)
        o = MO.newton_schulz(m, steps=8)
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.3 and s.min() > 0.5, (shape, s.min().item(), s.max().item())
        u, _, vt = torch.linalg.svd(m, full_matrices=False)
        cos = torch.nn.functional.cosine_similarity((u @ vt).flatten(), o.flatten(), dim=0)
        assert cos > 0.98


def _train(optimizer, iters=8, **kw):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=128,
                           params_dtype="fp32", seq_length=32)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=32, train_iters=iters, lr=kw.pop("lr", 2e-2),
                     lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1, optimizer=optimizer,
                     use_distributed_optimizer=optimizer == "adam", data_seed=3, **kw)
    torch.manual_seed(0)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    # a fixed batch so that the loss has to go down
    fixed = tr.stager.next_step()
    tr.stager.next_step = lambda: fixed
    tr.stager.prefetch = lambda: None
    return tr, tr.train()


def test_sgd_and_muon_reduce_the_loss_on_a_fixed_batch():
    for name, lr in (("sgd", 0.3), ("muon", 2e-2), ("adam", 1e-2)):
        _, losses = _train(name, lr=lr)
        assert losses[-1] < losses[0] - 0.3, (name, losses)


def test_evaluation_and_tokenizer():
    from primus_b200.engine import tokenizer as T

    tr, _ = _train("adam", iters=2, eval_interval=1, eval_iters=2)
    assert "validation_loss" in tr.last_metrics and tr.last_metrics["validation_loss"] > 0
    tok = T.build_tokenizer("NullTokenizer", vocab_size=1000, make_vocab_size_divisible_by=128)
    assert tok.vocab_size == 1001 and tok.eod == 1000 and tok.padded_vocab_size == 1024
    assert tok.tokenize("5 17 999") == [5, 17, 999] and tok.detokenize([1, 2]) == "1 2"
    import pytest
    with pytest.raises(ValueError):
        T.build_tokenizer("Llama3Tokenizer")


def test_chunked_linear_cross_entropy_matches_full():
    """Same loss trajectory with and without the chunked linear + cross-entropy path."""
    import dataclasses

    res = {}
    for chunk in (0, 24):
        from primus_b200.engine.trainer import TrainConfig, Trainer
        from primus_b200.models.config import TransformerConfig
        from primus_b200.parallel import state as ps

        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=128,
                               params_dtype="fp32", seq_length=32, cross_entropy_chunk_tokens=chunk)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=32, train_iters=4, lr=1e-2,
                         lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1)
        torch.manual_seed(0)
        tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
        res[chunk] = tr.train()
    assert all(abs(a - b) <= 1e-4 * max(1.0, abs(a)) for a, b in zip(res[0], res[24])), res


def test_profiler_trace_and_metrics_jsonl(tmp_path):
    import json

    tr, _ = _train("adam", iters=5, profile=True, profile_step_start=2, profile_step_end=3,
                   tensorboard_dir=str(tmp_path), exp_name="unit")
    lines = [json.loads(l) for l in (tmp_path / "metrics.jsonl").read_text().splitlines()]
    assert [l["iteration"] for l in lines] == [1, 2, 3, 4, 5]
    assert {"loss", "tokens_per_s_gpu", "grad_norm", "lr"} <= set(lines[0])
    traces = list((tmp_path / "profiler").glob("primus-b200-exp[[]unit[]]-rank[[]0[]].*.pt.trace.json"))
    assert len(traces) == 1 and traces[0].stat().st_size > 1000


def test_logit_softcapping_bounds_the_logits_and_trains():
    """final_logit_softcapping: logits stay inside (-cap, cap) and the model still trains; the attention variant is
    also available inside attention."""
    import pytest

    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import fused

    x = torch.randn(8, 16) * 50
    y = fused.softcap(x, 30.0)
    assert y.abs().max() < 30.0 and torch.allclose(y, torch.tanh(x / 30.0) * 30.0)
    assert fused.softcap(x, None) is x
    # soft-capped attention scores: the reference path bounds them, and a huge cap reproduces plain attention
    from primus_b200.ops import attention as A

    q, k, v = torch.randn(32, 2, 16) * 4, torch.randn(32, 2, 16) * 4, torch.randn(32, 2, 16)
    plain = A.attention_ref(q, k, v, 1, True)[0]
    assert torch.allclose(A.attention_ref(q, k, v, 1, True, softcap=1e6)[0], plain, atol=1e-4)
    assert not torch.allclose(A.attention_ref(q, k, v, 1, True, softcap=2.0)[0], plain, atol=1e-3)
    cfg = TransformerConfig(num_layers=1, hidden_size=64, num_attention_heads=4, attn_logit_softcapping=50.0)
    assert cfg.attn_logit_softcapping == 50.0


def test_multi_token_prediction_adds_a_trained_auxiliary_loss():
    """mtp_num_layers: extra depths share the embedding and the output head, add scale / D * CE to the loss, receive
    gradients, and the FLOPs model counts them."""
    from primus_b200.engine import schedules
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    kw = dict(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=128,
              params_dtype="fp32", seq_length=32)
    torch.manual_seed(0)
    base = GPTModel(TransformerConfig(**kw), "cpu")
    torch.manual_seed(0)
    cfg = TransformerConfig(**kw, mtp_num_layers=2, mtp_loss_scaling_factor=0.3)
    m = GPTModel(cfg, "cpu")
    names = [n for n, _ in m.named_parameters()]
    assert "mtp.layers.1.eh_proj.weight" in names and "mtp.layers.0.transformer_layer.mlp.linear_fc2.weight" in names
    tokens = torch.randint(0, 128, (2, 32))
    labels = torch.roll(tokens, -1, 1)
    w = torch.full((2, 32), 1.0 / 64)
    main = base(tokens, labels, loss_weights=w, unit_upstream=True)
    total = m(tokens, labels, loss_weights=w, unit_upstream=True)
    aux = (total - main).item()
    # two depths of ~ln(128) each, weighted 0.3 / 2, with 1 and 2 target-less positions per sequence
    assert 0.2 * 4.85 < aux < 0.4 * 4.85, aux
    total.backward()
    assert m.mtp.layers[1].eh_proj.weight.grad.abs().sum() > 0
    assert m.embedding.word_embeddings.weight.grad.abs().sum() > 0
    assert schedules.model_flops_per_token(cfg, 32) > schedules.model_flops_per_token(TransformerConfig(**kw), 32)


def test_sliding_window_and_sink_attention_in_the_model():
    """window_size / window_attn_skip_freq pick the window per layer, softmax_type learnable adds a trained per-head
    sink; a window at least as long as the sequence without sinks reproduces full attention."""
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    kw = dict(num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=128,
              params_dtype="fp32", seq_length=32)
    cfg = TransformerConfig(**kw, window_size=(7, 0), window_attn_skip_freq=2, softmax_type="learnable")
    assert [cfg.layer_window(i) for i in range(4)] == [8, 0, 8, 0]
    torch.manual_seed(0)
    m = GPTModel(cfg, "cpu")
    tokens = torch.randint(0, 128, (2, 32))
    labels = torch.roll(tokens, -1, 1)
    w = torch.full((2, 32), 1.0 / 64)
    loss = m(tokens, labels, loss_weights=w, unit_upstream=True)
    loss.backward()
    g = m.decoder.layers["0"].self_attention.core_attention.softmax_offset.grad
    assert g is not None and g.abs().sum() > 0
    torch.manual_seed(0)
    full = GPTModel(TransformerConfig(**kw), "cpu")
    torch.manual_seed(0)
    wide = GPTModel(TransformerConfig(**kw, window_size=32), "cpu")
    a = full(tokens, labels, loss_weights=w, unit_upstream=True)
    b = wide(tokens, labels, loss_weights=w, unit_upstream=True)
    assert torch.allclose(a, b, atol=1e-6)
    torch.manual_seed(0)
    narrow = GPTModel(TransformerConfig(**kw, window_size=4), "cpu")
    c = narrow(tokens, labels, loss_weights=w, unit_upstream=True)
    assert abs(c.item() - a.item()) > 1e-6


def test_precision_aware_optimizer_keeps_bf16_moments():
    """use_precision_aware_optimizer with bf16 moments: states are bf16, master weights fp32, and training follows
    the fp32-moment run closely."""
    tr32, l32 = _train("adam", iters=6, lr=1e-2)
    tr16, l16 = _train("adam", iters=6, lr=1e-2, use_precision_aware_optimizer=True, exp_avg_dtype="bf16",
                       exp_avg_sq_dtype="bf16")
    st = tr16.optimizer.state[0]
    assert st["m"].dtype == torch.bfloat16 and st["v"].dtype == torch.bfloat16 and st["master"].dtype == torch.float32
    assert tr32.optimizer.state[0]["m"].dtype == torch.float32
    assert all(abs(a - b) < 0.05 for a, b in zip(l32, l16)), (l32, l16)
    assert l16[-1] < l16[0] - 0.3


def test_step_timers_report_per_phase_times():
    logs = []
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, vocab_size=128,
                           params_dtype="fp32", seq_length=32)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=32, train_iters=2, log_interval=1,
                     timing_log_level=2, timing_log_option="minmax")
    Trainer(mc, tc, device="cpu", log_fn=logs.append).train()
    text = "\\n".join(logs)
    assert "(min, max) time across ranks (ms):" in text
    for name in ("forward-backward", "optimizer", "all-grads-sync", "batch-generator"):
        assert name in text, name
    quiet = []
    tc.timing_log_level = 0
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    Trainer(mc, tc, device="cpu", log_fn=quiet.append).train()
    assert "time across ranks" not in "\\n".join(quiet)


def test_expert_bias_moves_towards_balanced_load():
    """moe_router_enable_expert_bias: after every step the bias of over-used experts goes down and that of
    under-used ones up by the update rate, and the token counter restarts."""
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=1, moe=True)
    mc.moe_router_enable_expert_bias, mc.moe_router_score_function = True, "sigmoid"
    mc.moe_router_bias_update_rate = 0.01
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    layer = next(m for m in tr.model.modules() if hasattr(m, "update_expert_bias"))
    seen = {}
    orig = layer.update_expert_bias

    def spy(groups=()):
        seen["load"] = layer.router.local_tokens_per_expert.clone()
        orig(groups)

    layer.update_expert_bias = spy
    tr.train()
    load, bias = seen["load"], layer.router.expert_bias
    assert load.sum() == 4 * 32 * mc.moe_router_topk            # every routed copy of the global batch was counted
    assert torch.equal(bias, 0.01 * torch.sign(load.mean() - load))
    assert layer.router.local_tokens_per_expert.abs().sum() == 0


def test_llama3_rope_scaling_and_a_llama4_style_model():
    """use_rope_scaling stretches only the long wavelengths (Llama-3.x rule); a Llama-4-style layer stack (top-1 routed
    experts with the softmax taken before the top-k, a shared expert, dense and routed layers alternating, QK-norm)
    builds from the preset's switches and trains."""
    import math

    from primus_b200.core.config import presets
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.ops import fused
    from primus_b200.parallel import state as ps

    d, theta, factor, orig = 128, 500000.0, 8.0, 8192
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    got = fused.llama3_scale_frequencies(inv, factor, 1.0, 4.0, orig)
    for f0, f1 in zip(inv.tolist(), got.tolist()):
        wl = 2 * math.pi / f0
        if wl < orig / 4.0:
            want = f0
        elif wl > orig / 1.0:
            want = f0 / factor
        else:
            s = (orig / wl - 1.0) / (4.0 - 1.0)
            want = (1 - s) * f0 / factor + s * f0
        assert abs(f1 - want) <= 1e-6 * want
    assert (got < inv).any() and (got == inv).any()
    _, sin = fused.rope_tables(16, d, theta, "cpu", 1.0, dict(factor=factor))
    _, sin0 = fused.rope_tables(16, d, theta, "cpu")
    assert torch.equal(sin[:, 0], sin0[:, 0]) and torch.allclose(sin[:, -1] * factor, sin0[:, -1], rtol=1e-4)

    preset = presets.load_preset("llama4_17B128E", "models")
    assert preset["moe_layer_freq"] == 2 and preset["num_experts"] == 128 and preset["moe_router_topk"] == 1
    scout = presets.load_preset("llama4_17B16E", "models")
    assert scout["use_rope_scaling"] and scout["rope_scaling_factor"] == 16.0 and scout["qk_layernorm"]

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    cfg = TransformerConfig(num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                            vocab_size=128, params_dtype="fp32", seq_length=32, qk_layernorm=True, use_rope_scaling=True,
                            rope_scaling_factor=16.0, rope_scaling_original_max_position=16, num_experts=8,
                            moe_router_topk=1, moe_router_pre_softmax=True, moe_layer_freq=2, moe_ffn_hidden_size=64,
                            moe_shared_expert_intermediate_size=64, moe_aux_loss_coeff=0.001)
    assert cfg.moe_layer_pattern == [1, 0, 1, 0]
    torch.manual_seed(0)
    m = GPTModel(cfg, "cpu")
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    tokens = torch.randint(0, 128, (2, 32))
    labels = torch.roll(tokens, -1, 1)
    w = torch.full((2, 32), 1.0 / 64)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = m(tokens, labels, loss_weights=w, unit_upstream=True)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.3


def test_grad_spike_threshold_skips_the_step():
    """``odc_grad_spike_threshold``: a step whose global gradient norm exceeds the threshold updates nothing."""
    import torch

    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    def run(threshold):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                               vocab_size=256, params_dtype="fp32", make_vocab_size_divisible_by=64)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=1, lr=1e-2,
                         lr_decay_style="constant", clip_grad=0.0)
        torch.manual_seed(0)
        tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
        tr.optimizer.grad_spike_threshold = threshold
        before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
        tr.train(1)
        moved = any(not torch.equal(p, before[n]) for n, p in tr.model.named_parameters())
        return moved, float(tr.optimizer.grad_norm)

    moved, norm = run(0.0)
    assert moved and norm > 0
    assert run(norm * 0.5)[0] is False          # the norm is above the threshold: step skipped
    assert run(norm * 2.0)[0] is True


def test_grad_sanitize_zeroes_non_finite_entries_instead_of_skipping_the_step():
    """``sft_grad_sanitize``: a NaN / Inf in the gradient buffer makes the plain optimizer skip the whole step; with the
    sanitiser only the poisoned elements lose their update."""
    import torch

    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    def run(sanitize):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                               vocab_size=256, params_dtype="fp32", make_vocab_size_divisible_by=64)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=2, seq_length=32, train_iters=1, lr=1e-2,
                         lr_decay_style="constant", sft_grad_sanitize=sanitize)
        torch.manual_seed(0)
        tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
        before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
        # poison two gradient entries right before the optimizer looks at them
        orig = tr.optimizer.compute_grad_norm

        def poisoned():
            g = tr.buffers[0].grad_data
            g[5], g[77] = float("nan"), float("inf")
            return orig()

        tr.optimizer.compute_grad_norm = poisoned
        tr.train(1)
        moved = sum(int(not torch.equal(p, before[n])) for n, p in tr.model.named_parameters())
        return moved, int(tr.optimizer.sanitized_count), float(tr.optimizer.grad_norm)

    moved, count, norm = run(False)
    assert moved == 0 and count == 0                      # non-finite norm: the step is skipped
    moved, count, norm = run(True)
    assert moved > 0 and count == 2 and norm == norm and norm < float("inf")


def test_mlperf_log_events_order_and_convergence_stop(tmp_path):
    """``mlperf_mode``: header, init / run / block / eval intervals in the order the compliance checker expects, tracked
    stats per logged step, and the run ends with status success at the first evaluation that reaches the target."""
    import json

    from primus_b200.engine.mlperf_logging import PREFIX, MLPerfLogger, ThroughputClock
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    t = [0.0]
    clock = ThroughputClock(8, now=lambda: t[0])
    clock.begin(); t[0] = 2.0; clock.step(4); clock.pause(); t[0] = 5.0; clock.resume(); t[0] = 6.0
    assert clock.samples_per_s() == 32 / 3.0 and clock.samples_per_s(include_eval=True) == 32 / 6.0

    def run(target):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=6, layers=2, extra_tc=dict(
            mlperf_mode=True, mlperf_target_eval_loss=target, eval_interval=2, eval_iters=1,
            mlperf_log_path=str(tmp_path / f"mllog_{target}.txt")))
        lines = []
        tr = Trainer(mc, tc, device="cpu", log_fn=lines.append)
        losses = tr.train()
        ps.destroy_model_parallel()
        ev = [json.loads(l[len(PREFIX):]) for l in lines if l.startswith(PREFIX)]
        assert [json.loads(l[len(PREFIX):]) for l in open(tc.mlperf_log_path)] == ev
        return losses, ev

    losses, ev = run(100.0)                 # any loss is below this target: the first evaluation ends the run
    keys = [e["key"] for e in ev]
    assert len(losses) == 2 and keys[-1] == "run_stop" and ev[-1]["metadata"]["status"] == "success"
    assert keys[0] == "init_start" and keys.index("submission_benchmark") < keys.index("init_stop") < keys.index("run_start")
    order = [k for k in keys if k in ("init_stop", "run_start", "block_start", "block_stop", "eval_start", "eval_accuracy",
                                      "eval_stop", "run_stop")]
    assert order == ["init_stop", "run_start", "block_start", "block_stop", "eval_start", "eval_accuracy", "eval_stop", "run_stop"]
    assert keys.count("tracked_stats") == 2 and ev[keys.index("global_batch_size")]["value"] == 4
    acc = ev[keys.index("eval_accuracy")]
    assert acc["metadata"]["samples_count"] == 8 and acc["value"] > 0 and acc["event_type"] == "POINT_IN_TIME"
    assert all(set(e) == {"namespace", "time_ms", "event_type", "key", "value", "metadata"} for e in ev)
    losses, ev = run(0.001)                 # never reached: all iterations run, status aborted
    keys = [e["key"] for e in ev]
    assert len(losses) == 6 and keys.count("eval_accuracy") == 3 and ev[-1]["metadata"]["status"] == "aborted"
    assert keys.count("block_start") == 4 and keys.count("block_stop") == 3
    lg = MLPerfLogger("x", 4, enabled=False, sink=lambda l: (_ for _ in ()).throw(AssertionError("disabled logger wrote")))
    lg.log_init(1); lg.run_start(); lg.on_step(1, 1.0, 1e-3); lg.run_stop(True, 1)


def test_schedule_keys_reach_the_scheduler():
    """Warm-up fraction / start value, the WSD anneal and the weight-decay ramp are read from the training config."""
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=100, layers=2, lr=1.0, extra_tc=dict(
        lr_warmup_fraction=0.1, lr_warmup_init=0.2, lr_decay_iters=100, min_lr=0.0, lr_wsd_decay_iters=20,
        lr_wsd_decay_style="linear", start_weight_decay=0.0, end_weight_decay=0.2, weight_decay_incr_style="linear"))
    tc.lr_decay_style, tc.weight_decay = "WSD", 0.2
    s = Trainer(mc, tc, device="cpu", log_fn=lambda m: None).scheduler
    assert s.warmup_iters == 10 and abs(s.get_lr(5) - 0.6) < 1e-9 and s.get_lr(10) == 1.0      # from 0.2 to 1.0 in 10 steps
    assert s.get_lr(80) == 1.0 and abs(s.get_lr(90) - 0.5) < 1e-9 and s.get_lr(100) == 0.0     # stable, then a linear anneal
    assert abs(s.get_wd(50) - 0.1) < 1e-9 and s.get_wd(100) == 0.2
    ps.destroy_model_parallel()


def test_run_control_keys(tmp_path):
    """iterations_to_skip, skip_train, ckpt_step, override_opt_param_scheduler, save_retain_interval, pretrained_checkpoint,
    exit_on_missing_checkpoint, log_params_norm / log_num_zeros_in_grad, manual_gc_interval."""
    import os

    import pytest

    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    def make(iters=6, lr=1e-2, **extra):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, layers=2, lr=lr, extra_tc=extra)
        logs = []
        tr = Trainer(mc, tc, device="cpu", log_fn=logs.append)
        return tr, logs

    try:
        ref, _ = make()
        ref_losses = ref.train()
        sk, logs = make(iterations_to_skip=[2], log_params_norm=True, log_num_zeros_in_grad=True, manual_gc_interval=2)
        before = [p.detach().clone() for p in sk.model.parameters()]
        l1 = sk.train(1)
        mid = [p.detach().clone() for p in sk.model.parameters()]
        l2 = sk.train(1)                                      # the listed iteration: batch read, nothing updated
        assert l1[0] == ref_losses[0] and l2[0] == 0.0 and sk.iteration == 2
        assert any(not torch.equal(a, b) for a, b in zip(before, mid))
        assert all(torch.equal(a, b) for a, b in zip(mid, sk.model.parameters()))
        assert sk.stager.state_dict()["consumed_samples"] == 8 and any("iterations_to_skip" in m for m in logs)
        assert sk.last_metrics["params_norm"] > 0 and "num_zeros_in_grad" in sk.last_metrics
        assert any("params norm:" in m and "num zeros:" in m for m in logs)
        # checkpoints every 1 step, retained every 2: 1 and 3 go once a newer one exists
        root = str(tmp_path / "ck")
        a, _ = make(save=root, save_interval=1, save_retain_interval=2)
        a.train(5)
        assert sorted(n for n in os.listdir(root) if n.startswith("iter_")) == ["iter_0000002", "iter_0000004", "iter_0000005"]
        b, logs = make(ckpt_step=2, lr=5e-3)
        assert b.load_checkpoint(root) == 2 and b.scheduler.max_lr == 5e-3 and b.scheduler.num_iters == 2
        assert any("another schedule" in m and "this run's" in m for m in logs)   # this run's schedule, and it says so
        c, _ = make(lr=5e-3, use_checkpoint_opt_param_scheduler=True)
        assert c.load_checkpoint(root) == 5 and c.scheduler.max_lr == 1e-2        # the checkpoint's schedule on request
        with pytest.raises(FileNotFoundError):
            make(ckpt_step=3)[0].load_checkpoint(root)
        # nothing under load: weights from pretrained_checkpoint (iteration 0, fresh optimizer), or a clean stop
        empty = str(tmp_path / "empty")
        os.makedirs(empty)
        d, logs = make(pretrained_checkpoint=root)
        assert d.load_checkpoint(empty) == 0 and d.iteration == 0 and any("starting from the weights" in m for m in logs)
        assert all(torch.equal(x, y) for x, y in zip(d.model.parameters(), a.model.parameters()))
        with pytest.raises(SystemExit):
            make(exit_on_missing_checkpoint=True)[0].load_checkpoint(empty)
        e, logs = make(skip_train=True, eval_iters=1)
        assert e.train() == [] and e.iteration == 0 and any("validation loss" in m for m in logs)
    finally:
        ps.destroy_model_parallel()


def test_decoupled_and_head_learning_rates():
    """``decoupled_lr``: embeddings and output layer follow their own learning rate; ``head_lr_mult`` scales the output
    layer's.  With learning rate 0 for the rest, only those parameters move."""
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    def moved(**extra):
        ps.destroy_model_parallel()
        ps.initialize_model_parallel()
        mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=2, layers=2, lr=0.0, extra_tc=extra)
        tr = Trainer(mc, tc, device="cpu", log_fn=lambda m: None)
        before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
        tr.train()
        return {n for n, p in tr.model.named_parameters() if not torch.equal(p, before[n])}, tr

    try:
        assert moved()[0] == set()
        names, tr = moved(decoupled_lr=1e-2)
        assert names == {"embedding.word_embeddings.weight", "output_layer.weight"}
        assert tr._decoupled_scheduler.max_lr == 1e-2 and tr._decoupled_scheduler.decay_style == tr.scheduler.decay_style
        groups = {g for st in tr.optimizer.state for *_, g in st["wd_ranges"]}
        assert groups == {0, 1}
        names, _ = moved(decoupled_lr=1e-2, head_lr_mult=0.0)
        assert names == {"embedding.word_embeddings.weight"}
        # a multiplier on the head alone: compare the size of its update with and without
        def head_delta(**extra):
            ps.destroy_model_parallel()
            ps.initialize_model_parallel()
            mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=1, layers=2, lr=1e-3, extra_tc=extra)
            tr = Trainer(mc, tc, device="cpu", log_fn=lambda m: None)
            w0 = tr.model.output_layer.weight.detach().clone()
            tr.train()
            return (tr.model.output_layer.weight - w0).abs().mean().item()
        assert 2.5 < head_delta(head_lr_mult=3.0) / head_delta() < 3.5
    finally:
        ps.destroy_model_parallel()
