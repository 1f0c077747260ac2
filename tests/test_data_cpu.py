"""Megatron-format indexed datasets: write / read round trip, sample construction, blending, trainer wiring."""
import os

import numpy as np
import torch

from primus_b200.engine import indexed_dataset as ID


def _corpus(tmp_path, name="corpus", n_docs=37, seed=0, vocab=500, eod=499):
    rng = np.random.default_rng(seed)
    docs = [np.append(rng.integers(0, vocab - 1, size=int(rng.integers(5, 90))), eod) for _ in range(n_docs)]
    prefix = str(tmp_path / name)
    ID.write_indexed_dataset(prefix, docs, dtype=np.uint16)
    return prefix, docs


def test_index_round_trip_and_header(tmp_path):
    prefix, docs = _corpus(tmp_path)
    with open(prefix + ".idx", "rb") as f:
        assert f.read(9) == b"MMIDIDX\x00\x00"
    ds = ID.MMapIndexedDataset(prefix)
    assert len(ds) == len(docs) and ds.dtype == np.uint16
    for i in (0, 5, len(docs) - 1):
        assert np.array_equal(ds[i], docs[i])
    assert np.array_equal(ds.get(3, 2, 3), docs[3][2:5])


def test_gpt_samples_cover_every_epoch_token_once(tmp_path):
    prefix, docs = _corpus(tmp_path)
    g = ID.GPTIndexedDataset(prefix, 32, seed=7, eod_token=499, eod_mask_loss=True, reset_position_ids=True)
    total = sum(len(d) for d in docs)
    assert g.samples_per_epoch == (total - 1) // 32
    a, b = g[0], g[1]
    assert a["tokens"].shape == (32,) and torch.equal(a["labels"][:-1], a["tokens"][1:])
    assert a["labels"][-1] == b["tokens"][0]                                   # neighbouring samples share one token
    # the stream of one epoch is a permutation of the documents
    stream = torch.cat([g[i]["tokens"] for i in range(g.samples_per_epoch)]).numpy()
    counts = np.bincount(stream, minlength=500)
    allc = np.bincount(np.concatenate(docs), minlength=500)
    assert (counts <= allc).all() and counts.sum() == g.samples_per_epoch * 32
    # loss mask and positions follow the end-of-document tokens
    eods = (a["tokens"] == 499).nonzero().flatten()
    assert (a["loss_mask"][eods] == 0).all()
    for e in eods.tolist():
        if e + 1 < 32:
            assert a["position_ids"][e + 1] == 0
    # another epoch is another order; the same index is reproducible
    assert not torch.equal(g[0]["tokens"], g[g.samples_per_epoch]["tokens"])
    assert torch.equal(ID.GPTIndexedDataset(prefix, 32, seed=7)[3]["tokens"], g[3]["tokens"])


def test_blending_follows_the_weights(tmp_path):
    p1, _ = _corpus(tmp_path, "a", seed=1)
    p2, _ = _corpus(tmp_path, "b", seed=2)
    ds = ID.build_gpt_dataset(f"0.75 {p1} 0.25 {p2}", 16)
    share = (ds.which[:4000] == 0).mean()
    assert abs(share - 0.75) < 0.01
    assert ds[0]["tokens"].shape == (16,) and ds[12345]["tokens"].shape == (16,)


def test_trainer_reads_an_indexed_corpus(tmp_path):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    prefix, _ = _corpus(tmp_path, n_docs=200, vocab=500)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=3)
    tc.mock_data, tc.data_path = False, prefix
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    losses = tr.train()
    assert len(losses) == 3 and all(np.isfinite(losses))


def test_worker_threads_keep_the_sample_order_and_resume_exactly():
    """``num_workers`` > 0 loads the host side of the next step on worker threads: same batches in the same order, and a
    checkpoint taken with a step in flight replays it."""
    import time

    import torch

    from primus_b200.engine.data import BatchStager, MicroBatchSampler

    class Slow:
        def __len__(self):
            return 1 << 30

        def __getitem__(self, i):
            time.sleep(0.002)
            return {"tokens": torch.full((4,), i), "labels": torch.full((4,), i + 1)}

    def run(workers, steps, consumed=0):
        st = BatchStager(Slow(), MicroBatchSampler(8, 2, 1, 0, consumed), "cpu", num_workers=workers)
        out = []
        for _ in range(steps):
            out.append([mb["tokens"][:, 0].tolist() for mb in st.next_step()])
            st.prefetch()
        return out, st

    plain, _ = run(0, 4)
    threaded, st = run(3, 4)
    assert plain == threaded and plain[1][0] == [8, 9]
    # four steps consumed; whatever is staged or in flight is not counted
    assert st.state_dict() == {"consumed_samples": 32}
    resumed, _ = run(3, 2, consumed=st.state_dict()["consumed_samples"])
    assert resumed == run(0, 6)[0][4:]
    st.load_state_dict({"consumed_samples": 8})
    assert [mb["tokens"][:, 0].tolist() for mb in st.next_step()] == plain[1]


def test_split_gives_disjoint_training_and_validation_samples(tmp_path):
    import numpy as np
    import torch

    from primus_b200.engine.trainer import split_view

    class Ten:
        def __len__(self):
            return 200

        def __getitem__(self, i):
            return {"tokens": torch.tensor([i])}

    tr, va = split_view(Ten(), "99,1,0", 0), split_view(Ten(), "99,1,0", 1)
    assert len(tr) == 198 and len(va) == 2 and int(tr[197]["tokens"]) == 197 and int(va[0]["tokens"]) == 198
    assert int(tr[198]["tokens"]) == 0 and int(va[5]["tokens"]) == 199                 # wraps inside its own share
    a, b = split_view(Ten(), "8,1,1", 1), split_view(Ten(), "8,1,1", 2)
    assert (a.lo, a.n, b.lo, b.n) == (160, 20, 180, 20)
    # through the trainer: the validation stream never touches the training share of a token file
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    path = str(tmp_path / "corpus.bin")
    np.arange(33 * 400, dtype=np.int32).tofile(path)          # sample i holds tokens [33 i, 33 i + 33): recognisable
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=2, layers=2, vocab=16384,
                         extra_tc=dict(mock_data=False, data_path=path, split="90,10,0", eval_iters=2))
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    t = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    n = len(t.stager.dataset.dataset)
    train_first = [int(mb["tokens"][0, 0]) for mb in t.stager.next_step()]
    valid_first = [int(mb["tokens"][0, 0]) for mb in t._eval_stager().next_step()]
    assert len(t.stager.dataset) == round(0.9 * n) and all(v >= 32 * round(0.9 * n) for v in valid_first)
    assert all(x < 32 * round(0.9 * n) for x in train_first)
    ps.destroy_model_parallel()


def test_batch_size_rampup(tmp_path):
    """``rampup_batch_size: [start, increment, samples]``: the global batch grows in equal stretches of the first samples;
    the trainer follows with its number of micro-batches and the stream stays resumable in the middle of the ramp."""
    import torch

    from primus_b200.engine.data import BatchStager, MicroBatchSampler, MockGPTDataset
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    s = MicroBatchSampler(16, 2, 2, 1, rampup=(4, 4, 48))          # 4 -> 8 -> 12 -> 16 over 48 samples: 16 samples each
    sizes, firsts = [], []
    for _ in range(10):
        mbs = s.next_global_batch()
        sizes.append(s.last_batch_size)
        firsts.append(mbs[0][0])
    assert sizes == [4, 4, 4, 4, 8, 8, 12, 12, 16, 16] and s.consumed == sum(sizes)
    assert firsts[0] == 2 and firsts[4] == 16 + 2                   # rank 1 of 2: the second micro-batch of every pair
    import pytest
    with pytest.raises(AssertionError):
        MicroBatchSampler(16, 2, 2, 0, rampup=(4, 5, 48))
    with pytest.raises(AssertionError):
        MicroBatchSampler(16, 4, 2, 0, rampup=(4, 4, 48))           # 4 is not a multiple of micro batch x dp = 8
    ds = MockGPTDataset(100, 8)
    st = BatchStager(ds, MicroBatchSampler(8, 2, 1, 0, rampup=(2, 2, 12)), "cpu", num_workers=2)
    seen = [len(st.next_step()) for _ in range(3)]
    assert seen == [1, 1, 2] and st.state_dict() == {"consumed_samples": 8}   # 2 + 2 + 4; what is in flight is not counted
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=8, mbs=2, iters=5, layers=2, extra_tc=dict(rampup_batch_size=[2, 2, 12]))
    logs = []
    tr = Trainer(mc, tc, device="cpu", log_fn=logs.append)
    counts = []
    tr.train(on_step=lambda t, lv: counts.append((t.num_microbatches, t.current_global_batch)))
    assert counts == [(1, 2), (1, 2), (2, 4), (3, 6), (4, 8)]        # stretches of 4 samples: 2, 2 | 4 | 6 | 8
    assert any("global batch size:     6" in m for m in logs)
    ps.destroy_model_parallel()


def test_data_subcommand_blend_inspect_and_pack(tmp_path, capsys):
    import argparse
    import json

    import numpy as np

    from primus_b200.cli.subcommands import data as D
    from primus_b200.engine.indexed_dataset import write_indexed_dataset

    def run(*argv):
        ap = argparse.ArgumentParser()
        D.register_subcommand(ap.add_subparsers(dest="cmd"))
        a = ap.parse_args(["data", *argv])
        assert D.run(a, []) == 0
        return capsys.readouterr().out

    rng = np.random.default_rng(0)
    for name, docs in (("a", 40), ("b", 10)):
        write_indexed_dataset(str(tmp_path / name), [rng.integers(0, 100, size=100).astype(np.int32) for _ in range(docs)],
                              dtype=np.int32)
    info = json.loads(run("inspect", "--path", str(tmp_path / "a"), "--seq-length", "32"))
    assert info["format"] == "megatron" and info["documents"] == 40 and info["tokens"] == 4000 and info["samples"] == 124
    plan = json.loads(run("blend", "--data-path", f"3 {tmp_path / 'a'} 1 {tmp_path / 'b'}", "--seq-length", "32",
                          "--samples", "400"))
    a, b = plan["datasets"]
    assert (a["weight"], b["weight"]) == (0.75, 0.25) and a["samples_drawn"] == 300 and b["samples_drawn"] == 100
    assert a["epochs"] == round(300 / 124, 3) and b["epochs"] == round(100 / 31, 3)      # the small corpus repeats more
    recs = tmp_path / "sft.jsonl"
    recs.write_text("\n".join(json.dumps({"instruction": f"add {i}", "input": "", "output": str(i) * 5}) for i in range(30)))
    out = run("pack-sft", "--input", str(recs), "--seq-length", "256", "--cache-dir", str(tmp_path / "cache"))
    res = json.loads(out.strip().splitlines()[-1])
    assert res["packs"] >= 1 and len(list((tmp_path / "cache").iterdir())) == 1
    again = run("pack-sft", "--input", str(recs), "--seq-length", "256", "--cache-dir", str(tmp_path / "cache"))
    assert json.loads(again.strip().splitlines()[-1]) == res and len(list((tmp_path / "cache").iterdir())) == 1
