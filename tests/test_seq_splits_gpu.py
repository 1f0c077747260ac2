"""Sequence splits on the GPU path: chunk queries against the kept key prefix through the offset form of the attention
kernels; the losses must follow the unsplit run."""
import pytest
import torch

from primus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _run(splits):
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2, num_query_groups=1,
                           kv_channels=128, vocab_size=1024, params_dtype="bf16", seq_length=512)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_length=512, train_iters=4, lr=1e-3,
                     lr_decay_style="constant", num_seq_splits=splits)
    torch.manual_seed(0)
    tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
    losses = tr.train()
    torch.cuda.synchronize()
    _lib.check_status()
    return losses


def test_chunked_sequence_follows_the_whole_sequence_on_gpu():
    ref = _run(1)
    for splits in (2, 4):
        got = _run(splits)
        assert all(abs(a - b) <= 5e-3 * abs(a) for a, b in zip(ref, got)), (splits, ref, got)
