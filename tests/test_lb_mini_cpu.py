"""LB-Mini: balanced dealing of variable-length samples over data-parallel ranks with per-rank micro-batch counts."""
import json
import random

import torch

from primus_b200.engine import lb_mini as LB
from tests.mp_utils import run_ranks


def test_karmarkar_karp_balances_and_covers():
    rng = random.Random(0)
    costs = [float(rng.choice([30, 60, 120, 500, 900, 4000])) for _ in range(64)]
    for k in (2, 4, 8):
        parts = LB.karmarkar_karp(costs, k)
        assert sorted(i for p in parts for i in p) == list(range(64))
        naive_k = [[i for i in range(64) if i % k == r] for r in range(k)]
        assert LB.partition_spread(costs, parts) < min(0.15, LB.partition_spread(costs, naive_k))
        eq = LB.karmarkar_karp(costs, k, equal_size=True)
        assert all(len(p) == 64 // k for p in eq) and sorted(i for p in eq for i in p) == list(range(64))
    naive = [[i for i in range(64) if i % 4 == r] for r in range(4)]
    assert LB.partition_spread(costs, LB.karmarkar_karp(costs, 4)) < LB.partition_spread(costs, naive)


def test_rearrange_gives_variable_counts_and_respects_cap():
    lengths = [4000] * 3 + [100] * 40 + [900] * 5
    seen, counts = [], []
    for r in range(4):
        mbs, stats = LB.rearrange_micro_batches(lengths, 4, r, 4096)
        counts.append(len(mbs))
        for mb in mbs:
            assert sum(min(lengths[i], 4096) for i in mb) <= 4096
            seen += mb
        assert stats["micro_batches_per_rank"][r] == len(mbs)
        assert stats["cost_spread"] < stats["naive_token_spread"]
    assert sorted(seen) == list(range(len(lengths)))
    same = [len(LB.rearrange_micro_batches(lengths, 4, r, 4096, same_num_in_dp=True)[0]) for r in range(4)]
    assert len(set(same)) == 1 and same[0] == max(counts)
    fit = LB.seq_costs_fit([100, 200], a=1.0, b=0.0, norm=100.0)
    assert fit == [1.0, 4.0]


def _records(n=24):
    rng = random.Random(1)
    return [{"instruction": "q" * rng.choice([3, 10, 40, 200]), "input": "", "output": "a" * rng.choice([2, 30, 120])}
            for _ in range(n)]


def _sft_worker(rank, world, lb, outp):
    from primus_b200.engine.lb_mini import LBMiniStager
    from primus_b200.engine.sft import ByteTokenizer, SFTDataset
    from primus_b200.engine.data import BatchStager, MicroBatchSampler
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    st = ps.get_state()
    mc = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
                           vocab_size=320, params_dtype="fp32", make_vocab_size_divisible_by=64)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=8, seq_length=512, train_iters=3, lr=1e-3,
                     lr_decay_style="constant", log_interval=1, calculate_per_token_loss=False)
    torch.manual_seed(3)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    ds = SFTDataset(_records(), ByteTokenizer(), 512, "alpaca", True)
    logs = []
    if lb:
        tr.stager = LBMiniStager(ds, 8, st.dp, st.dp_rank, "cpu", 512, log=logs.append)
    else:   # one sample per micro-batch, dealt round-robin, normalised by the same mini-batch token count
        tr.stager = LBMiniStager(ds, 8, st.dp, st.dp_rank, "cpu", 512, log=None)
        tr.stager.same_num_in_dp = True
    tr.sampler = tr.stager.sampler
    tr.use_position_ids = True
    counts = []
    orig = tr.stager.next_step

    def counted():
        mbs = orig()
        counts.append(len(mbs))
        return mbs
    tr.stager.next_step = counted
    losses = tr.train(3)
    json.dump({"losses": losses, "counts": counts, "stats": tr.stager.last_stats}, open(f"{outp}.{rank}", "w"))


def test_sft_training_with_lb_mini_dp2(tmp_path):
    """Two data-parallel ranks with different numbers of micro-batches per step train in lockstep; the trajectory
    equals the equal-count variant of the same dealing (the loss normalisation does not depend on the dealing)."""
    a, b = str(tmp_path / "lb"), str(tmp_path / "same")
    run_ranks(_sft_worker, 2, "gloo", args=(True, a), timeout=300)
    run_ranks(_sft_worker, 2, "gloo", args=(False, b), timeout=300)
    r0, r1 = json.load(open(a + ".0")), json.load(open(a + ".1"))
    s0 = json.load(open(b + ".0"))
    assert r0["losses"] == r1["losses"] and all(0 < l < 10 for l in r0["losses"])
    assert r0["stats"]["cost_spread"] <= r0["stats"]["naive_token_spread"] + 1e-9
    for x, y in zip(r0["losses"], s0["losses"]):
        assert abs(x - y) < 1e-4 * max(1.0, abs(y))
