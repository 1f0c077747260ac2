"""Trainer-level checks on a GPU: bitwise run-to-run reproducibility (the reference compares logged losses of two
deterministic runs string by string, tests/trainer/test_megatron_trainer.py:869-966) and checkpoint resume."""
import pytest
import torch

from primus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _run(kind: str, iters: int, save=None, load=None, resume_iters=None, **model_kw):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    kw = dict(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2, num_query_groups=2,
              vocab_size=1024, params_dtype="bf16", seq_length=256)
    if kind == "mxfp8":
        kw.update(fp8="e4m3", fp8_recipe="mxfp8")
    if kind == "moe":
        kw.update(num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=256, moe_layer_freq=[0, 1],
                  moe_aux_loss_coeff=1e-2)
    kw.update(model_kw)
    try:
        mc = TransformerConfig(**kw)
        tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=mc.seq_length, train_iters=iters, lr=2e-3,
                         lr_decay_style="constant", weight_decay=0.01, clip_grad=1.0, log_interval=1, save=save,
                         load=load, save_interval=iters if save else None)
        torch.manual_seed(0)
        tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
        if load:
            assert tr.load_checkpoint(load) > 0
        losses = tr.train(resume_iters)
        torch.cuda.synchronize()
        _lib.check_status()
        return losses
    finally:
        gemm.set_fp8_recipe(None)


@pytest.mark.parametrize("kind", ["bf16", "mxfp8", "moe"])
def test_two_runs_log_identical_losses(kind):
    a = _run(kind, 5)
    b = _run(kind, 5)
    assert a == b, (a, b)


def test_resume_from_checkpoint_continues_bitwise(tmp_path):
    full = _run("bf16", 6)
    first = _run("bf16", 3, save=str(tmp_path / "ck"))
    rest = _run("bf16", 6, load=str(tmp_path / "ck"), resume_iters=3)
    assert first == full[:3]
    assert rest == full[3:], (rest, full[3:])


def test_activation_offload_changes_nothing_but_where_tensors_live():
    from primus_b200.engine import offload

    base = _run("bf16", 3, seq_length=2048)
    before = offload.STATS["offloaded_tensors"]
    off = _run("bf16", 3, seq_length=2048, cpu_offloading=True, cpu_offloading_num_layers=2)
    assert offload.STATS["offloaded_tensors"] > before and offload.STATS["offloaded_bytes"] > 0
    assert off == base, (off, base)
