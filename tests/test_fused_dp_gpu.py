"""Fused data-parallel optimizer (P2P reduce-scatter + AdamW + all-gather through symmetric memory) must follow
the NCCL path step for step (2 GPUs)."""
import json

import pytest
import torch

from tests.mp_utils import run_ranks

pytestmark = pytest.mark.gpu


def _worker(rank, world, fused, outp, extra=None):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import _lib
    from primus_b200.parallel import state as ps

    ps.initialize_model_parallel()
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1408, num_attention_heads=4,
                            num_query_groups=2, kv_channels=128, vocab_size=8192, params_dtype="bf16")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=256, train_iters=4, lr=1e-3,
                     lr_decay_style="constant", fused_dp_optimizer=fused, ddp_bucket_size=1_000_000, **(extra or {}))
    tr = Trainer(cfg, tc, device=f"cuda:{rank}", log_fn=lambda s: None)
    losses = tr.train(4)
    tr.finish_param_sync()
    torch.cuda.synchronize()
    _lib.check_status()
    checksum = float(sum(p.detach().float().abs().sum() for p in tr.model.parameters()))
    if rank == 0:
        json.dump({"losses": losses, "checksum": checksum, "symmetric": bool(tr.buffers[0].symmetric)}, open(outp, "w"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_dp_optimizer_matches_nccl(tmp_path):
    a, b = str(tmp_path / "nccl.json"), str(tmp_path / "fused.json")
    run_ranks(_worker, 2, "nccl", args=(False, a), timeout=240)
    run_ranks(_worker, 2, "nccl", args=(True, b), timeout=240)
    ra, rb = json.load(open(a)), json.load(open(b))
    assert rb["symmetric"] and not ra["symmetric"]
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) <= 2e-3 * max(1.0, abs(x)), (ra, rb)
    assert abs(ra["checksum"] - rb["checksum"]) <= 1e-3 * ra["checksum"]


VARIANTS = {
    "nccl_overlap": (False, dict(overlap_grad_reduce=True, overlap_param_gather=True), 1e-6),
    "fused_overlap": (True, dict(overlap_grad_reduce=True), 2e-3),
    "bf16_reduce": (False, dict(overlap_grad_reduce=True, grad_reduce_in_bf16=True), 2e-2),
    # parameter all-gather by copy-engine pulls on a side stream, with and without per-layer waits
    "copy_engine": (True, dict(overlap_grad_reduce=True, param_gather_copy_engine=True), 2e-3),
    "copy_engine_overlap": (True, dict(overlap_grad_reduce=True, param_gather_copy_engine=True,
                                       overlap_param_gather=True), 2e-3),
    # on-demand communication: gradients pushed into the owners' accumulators with peer atomics, parameters pulled
    "odc": (False, dict(enable_odc=True, overlap_grad_reduce=True), 2e-3),
}


@pytest.fixture(scope="module")
def plain_nccl_run(tmp_path_factory):
    base = str(tmp_path_factory.mktemp("dp_base") / "base.json")
    run_ranks(_worker, 2, "nccl", args=(False, base), timeout=240)
    return json.load(open(base))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_overlapped_variants_match_the_plain_nccl_path(name, plain_nccl_run, tmp_path):
    """Per-bucket overlap of the gradient reduction (NCCL and fused), bf16 on the wire, the asynchronous parameter
    all-gather with per-layer waits (NCCL or copy engines) and on-demand communication must not change the training
    trajectory."""
    ref = plain_nccl_run
    fused, extra, tol = VARIANTS[name]
    outp = str(tmp_path / f"{name}.json")
    run_ranks(_worker, 2, "nccl", args=(fused, outp, extra), timeout=240)
    got = json.load(open(outp))
    for x, y in zip(ref["losses"], got["losses"]):
        assert abs(x - y) <= tol * max(1.0, abs(x)), (name, ref, got)
    assert abs(ref["checksum"] - got["checksum"]) <= max(tol, 1e-3) * ref["checksum"], name


def _fsdp_worker(rank, world, fsdp, outp):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import _lib
    from primus_b200.parallel import state as ps

    ps.initialize_model_parallel()
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1408, num_attention_heads=4,
                            num_query_groups=2, kv_channels=128, vocab_size=8192, params_dtype="bf16")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=256, train_iters=4, lr=1e-3,
                     lr_decay_style="constant", use_torch_fsdp2=fsdp)
    torch.manual_seed(0)
    tr = Trainer(cfg, tc, device=f"cuda:{rank}", log_fn=lambda s: None)
    losses = tr.train(4)
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        json.dump({"losses": losses, "fsdp": bool(tr.fsdp)}, open(outp, "w"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp2_follows_the_distributed_optimizer(tmp_path):
    """Fully sharded run (torch fully_shard around this package's layers) vs the ZeRO-1 distributed optimizer."""
    a, b = str(tmp_path / "zero1.json"), str(tmp_path / "fsdp.json")
    run_ranks(_fsdp_worker, 2, "nccl", args=(False, a), timeout=240)
    run_ranks(_fsdp_worker, 2, "nccl", args=(True, b), timeout=240)
    ra, rb = json.load(open(a)), json.load(open(b))
    assert rb["fsdp"] and not ra["fsdp"]
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) <= 5e-3 * max(1.0, abs(x)), (ra, rb)
