"""MXFP8 recipe under tensor + sequence parallelism: the all-gathers move the quantised shards (values + block scales)
and must give bit-identical results to gathering bf16 and quantising the gathered tensor (2 GPUs)."""
import json

import pytest
import torch

from tests.mp_utils import run_ranks

pytestmark = pytest.mark.gpu


def _gather_worker(rank, world):
    import torch.distributed as dist

    from primus_b200.ops import _lib, fp8, gemm
    from primus_b200.parallel import fused_tp
    from primus_b200.parallel import tensor_parallel as tpc

    group = dist.group.WORLD
    torch.manual_seed(7 + rank)
    gemm.set_fp8_recipe("mxfp8")
    try:
        Tl, K, N = 256, 512, 384
        x = (torch.randn(Tl, K, device="cuda") * torch.exp(torch.randn(Tl, 1, device="cuda"))).bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        ph = fused_tp.all_gather_quantized(x, group, row=True, col=True)
        ref = fp8.quantize_mxfp8(tpc.all_gather_dim0(x, group), True, True)
        aq, asf = gemm._quantized(ph, "row")
        assert torch.equal(aq, ref.q_row) and torch.equal(asf, ref.sf_row)
        cq, csf = gemm._quantized(ph, "col")                      # the last consumer releases the table entry
        assert torch.equal(cq, ref.q_col) and torch.equal(csf, ref.sf_col)
        assert not gemm._PINNED
        out, g = fused_tp.ag_gemm(x, w, group)
        fused_tp.QUANTIZED_GATHER = False
        out_ref, _ = fused_tp.ag_gemm(x, w, group)
        fused_tp.QUANTIZED_GATHER = True
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(out, out_ref) and not gemm._PINNED
    finally:
        gemm.set_fp8_recipe(None)


def _train_worker(rank, world, quantized, outp):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import _lib
    from primus_b200.parallel import fused_tp
    from primus_b200.parallel import state as ps

    fused_tp.QUANTIZED_GATHER = quantized
    ps.initialize_model_parallel(tp=2)
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1536, num_attention_heads=4,
                            num_query_groups=2, kv_channels=128, vocab_size=8192, params_dtype="bf16",
                            tensor_model_parallel_size=2, sequence_parallel=True, fp8="e4m3", fp8_recipe="mxfp8")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=512, train_iters=4, lr=1e-3,
                     lr_decay_style="constant")
    tr = Trainer(cfg, tc, device=f"cuda:{rank}", log_fn=lambda s: None)
    losses = tr.train(4)
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        json.dump(losses, open(outp, "w"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_quantized_gather_is_bit_identical_to_quantising_the_gathered_tensor():
    run_ranks(_gather_worker, 2, "nccl", timeout=240)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_training_with_quantized_gathers_matches_bf16_gathers(tmp_path):
    a, b = str(tmp_path / "q.json"), str(tmp_path / "p.json")
    run_ranks(_train_worker, 2, "nccl", args=(True, a), timeout=240)
    run_ranks(_train_worker, 2, "nccl", args=(False, b), timeout=240)
    qa, pb = json.load(open(a)), json.load(open(b))
    assert qa == pb, (qa, pb)          # same quantised operands, same kernels: identical trajectories
