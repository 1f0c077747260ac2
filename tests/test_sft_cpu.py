"""SFT: formatters, answer-only masks, packing invariants, LoRA adapter training (base weights frozen, merge)."""
import json

import torch

from primus_b200.engine import sft as S


def test_formatters():
    p, a = S.format_alpaca({"instruction": "Add", "input": "1 2", "output": "3"})
    assert "### Input:\n1 2" in p and a == "3"
    p, a = S.format_alpaca({"instruction": "Say hi", "output": "hi"})
    assert "### Input" not in p
    p, a = S.format_squad({"context": "C", "question": "Q", "answers": {"text": ["A"]}})
    assert p.endswith("Answer:") and a == " A"
    p, a = S.FORMATTERS["chatml"]({"messages": [{"role": "user", "content": "u"}, {"role": "assistant", "content": "v"}]})
    assert p == "<|im_start|>user\nu<|im_end|>\n<|im_start|>assistant\n" and a == "v<|im_end|>\n"
    p, a = S.FORMATTERS["openai"]({"conversations": [{"from": "human", "value": "u"}, {"from": "gpt", "value": "v"}]})
    assert p == "user: u\nassistant: " and a == "v"


def _records(n=40):
    return [{"instruction": "repeat " + "x" * (i % 17), "output": "y" * (1 + i % 23)} for i in range(n)]


def test_answer_only_loss_mask_and_padding():
    ds = S.SFTDataset(_records(4), S.ByteTokenizer(), 512, "alpaca", True)
    it = ds[0]
    assert it["tokens"].shape == (512,) and it["loss_mask"].sum() > 0
    n_prompt = len(S.ByteTokenizer().encode(S.format_alpaca(_records(1)[0])[0]))
    assert it["loss_mask"][: n_prompt - 1].sum() == 0          # no loss on the prompt
    assert it["loss_mask"][n_prompt - 1] == 1                   # first answer token is predicted from the last prompt token
    full = S.SFTDataset(_records(4), S.ByteTokenizer(), 512, "alpaca", False)[0]
    assert full["loss_mask"].sum() > it["loss_mask"].sum()


def test_packing_invariants():
    lengths = [5, 300, 200, 512, 17, 100, 250, 250, 9]
    for algo in ("first_fit", "first_fit_decreasing", "first_fit_shuffle"):
        bins = S.pack_bins(lengths, 512, algo, seed=3)
        assert sorted(i for b in bins for i in b) == list(range(len(lengths)))
        assert all(sum(lengths[i] for i in b) <= 512 for b in bins)
    assert len(S.pack_bins(lengths, 512, "first_fit_decreasing")) <= len(S.pack_bins(lengths, 512, "first_fit"))
    ds = S.SFTDataset(_records(), S.ByteTokenizer(), 512, "alpaca", True)
    pk = S.PackedSFTDataset(ds)
    assert len(pk) < len(ds) and pk.packing_efficiency() > 0.5
    it = pk[0]
    starts = (it["position_ids"] == 0).nonzero().flatten()
    assert len(starts) >= 2                                     # several samples, positions restart


def test_lora_trains_adapters_only(tmp_path):
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps
    from tests import dist_workers as W

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=6)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    tr.lora = S.LoRAEngine(tr.model_chunks, rank=4, alpha=8.0, lr=5e-2)
    h = tr.lora.holders[0]
    base = h.base_weight.clone()
    emb = tr.model.embedding.word_embeddings.weight.detach().clone()
    losses = tr.train(6)
    assert torch.equal(h.base_weight, base)                               # frozen
    assert torch.equal(tr.model.embedding.word_embeddings.weight, emb)    # non-adapted parameters untouched
    assert h.lora.lora_b.abs().sum() > 0                                  # adapters moved
    assert not torch.equal(h.weight.detach(), base)                       # effective weight = base + BA
    assert torch.allclose(h.weight.detach(), base + h.lora.delta(), atol=1e-5)
    n = S.merge_lora(tr.model)
    assert n == len(tr.lora.holders) and not hasattr(h, "lora")
    assert any(".lora." in k for k in []) is False and len(losses) == 6


def test_sft_trainer_through_cli(tmp_path):
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    data = tmp_path / "sft.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in _records(16)))
    exp = tmp_path / "exp.yaml"
    exp.write_text(f"""
work_group: t
user_name: u
exp_name: sft
workspace: {tmp_path}/out
modules:
  post_trainer:
    config: sft_trainer.yaml
    model: llama_tiny.yaml
    overrides:
      train_iters: 2
      micro_batch_size: 2
      global_batch_size: 4
      seq_length: 128
      vocab_size: 512
      params_dtype: fp32
      sft_dataset_name: {data}
      sft_packing: true
      peft: lora
      lora_rank: 4
""")
    r = subprocess.run([sys.executable, "-m", "primus_b200.cli.main", "train", "posttrain", "--config", str(exp)],
                       capture_output=True, text=True, cwd=root, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Training completed." in r.stderr


def test_aligned_packing_and_document_boundaries():
    ds = S.SFTDataset(_records(), S.ByteTokenizer(), 512, "alpaca", True)
    pk = S.PackedSFTDataset(ds, align=128)
    it = pk[0]
    cu = [c for c in it["host_cu_seqlens"].tolist() if c >= 0]
    assert cu[0] == 0 and cu[-1] == 512 and all(c % 128 == 0 for c in cu) and cu == sorted(set(cu))
    # positions restart at every boundary that starts a sample; padding carries no loss
    for a in cu[:-1]:
        assert it["position_ids"][a] == 0 or it["loss_mask"][a:].sum() == 0
    assert len(it["host_cu_seqlens"]) == 512 // 128 + 2
    assert "host_cu_seqlens" not in S.PackedSFTDataset(ds, boundaries=False)[0]


def test_attention_stays_inside_each_packed_document():
    """A model run on two documents packed into one sequence (with their boundaries) gives each document the loss it
    gets when run alone; without the boundaries the second document sees the first and its loss changes."""
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    torch.manual_seed(0)
    m = GPTModel(TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4,
                                   vocab_size=128, params_dtype="fp32", seq_length=32), "cpu")
    a, b = torch.randint(0, 128, (1, 20)), torch.randint(0, 128, (1, 12))
    tok = torch.cat([a, b], 1)
    lab = torch.roll(tok, -1, 1)
    pos = torch.cat([torch.arange(20), torch.arange(12)]).view(1, 32)
    cu = torch.tensor([[0, 20, 32, -1]], dtype=torch.int32)
    packed = m(tok, lab, position_ids=pos, cu_seqlens=cu)                    # per-token losses [1, 32]
    alone_a = m(a, lab[:, :20], position_ids=pos[:, :20])
    alone_b = m(b, lab[:, 20:], position_ids=pos[:, 20:])
    assert torch.allclose(packed[:, :20], alone_a, atol=1e-5) and torch.allclose(packed[:, 20:], alone_b, atol=1e-5)
    leaky = m(tok, lab, position_ids=pos)
    assert torch.allclose(leaky[:, :20], alone_a, atol=1e-5) and not torch.allclose(leaky[:, 20:], alone_b, atol=1e-4)


def test_pack_cache_roundtrip_and_key(tmp_path, monkeypatch):
    """The packed dataset is built once, stored under a key that covers data file, tokenizer and packing settings, and
    loaded bit-identically afterwards."""
    import json as _json

    from primus_b200.engine import sft as S

    data = tmp_path / "d.jsonl"
    recs = [{"instruction": f"q{i} " * (i % 7 + 1), "input": "", "output": f"a{i} " * (i % 5 + 1)} for i in range(40)]
    data.write_text("\n".join(_json.dumps(r) for r in recs))
    monkeypatch.setenv("PRIMUS_PACK_CACHE_DIR", str(tmp_path / "cache"))
    tok = S.ByteTokenizer()
    logs = []
    a = S.load_or_build_packed(str(data), tok, 128, "alpaca", True, "first_fit_decreasing", 0, 1, True, log=logs.append)
    files = list((tmp_path / "cache").glob("packed_*.pt"))
    assert len(files) == 1 and "built and cached" in logs[-1]
    b = S.load_or_build_packed(str(data), tok, 128, "alpaca", True, "first_fit_decreasing", 0, 1, True, log=logs.append)
    assert "loaded from cache" in logs[-1] and len(a) == len(b) and a.bins == b.bins
    for i in range(len(a)):
        for k in a[i]:
            assert torch.equal(a[i][k], b[i][k]), (i, k)
    # another sequence length, algorithm or tokenizer is another entry
    S.load_or_build_packed(str(data), tok, 256, "alpaca", True, "first_fit_decreasing", 0, 1, True)
    S.load_or_build_packed(str(data), tok, 128, "alpaca", True, "first_fit", 0, 1, True)
    monkeypatch.setenv("PRIMUS_PACK_TOKENIZER_ID", "other-tokenizer")
    S.load_or_build_packed(str(data), tok, 128, "alpaca", True, "first_fit_decreasing", 0, 1, True)
    assert len(list((tmp_path / "cache").glob("packed_*.pt"))) == 4
    assert S.pack_cache_dir(str(tmp_path / "explicit")) == str(tmp_path / "explicit")


def test_mlperf_packed_directory_is_used_as_stored(tmp_path):
    """train.npy / packed_metadata.jsonl in the MLPerf layout: labels shifted inside each segment, no target across a
    segment start, positions restart, boundaries exported."""
    import json as _json

    import numpy as np

    from primus_b200.engine import sft as S

    L = 16
    packs = np.empty(2, dtype=object)
    packs[0] = {"input_ids": np.arange(100, 100 + L, dtype=np.int32), "loss_mask": [0] * 4 + [1] * 12, "seq_start_id": [0]}
    packs[1] = {"input_ids": np.arange(200, 200 + L, dtype=np.int32), "loss_mask": [0, 1] * 8, "seq_start_id": [0, 8]}
    np.save(tmp_path / "train.npy", packs, allow_pickle=True)
    np.save(tmp_path / "validation.npy", packs[:1], allow_pickle=True)
    (tmp_path / "packed_metadata.jsonl").write_text(_json.dumps([{"max_samples_per_bin": 2, "dataset_max_seqlen": L}]))
    assert S.is_mlperf_packed_dir(str(tmp_path)) and not S.is_mlperf_packed_dir(str(tmp_path / "train.npy"))
    ds = S.MLPerfPackedDataset(str(tmp_path))
    assert len(ds) == 2 and ds.seq_length == L
    a = ds[0]
    assert a["tokens"].tolist() == list(range(100, 116)) and a["labels"][:15].tolist() == list(range(101, 116))
    assert a["loss_mask"].tolist() == [0.0] * 3 + [1.0] * 12 + [0.0]          # shifted by one, last position has no target
    b = ds[1]
    assert b["position_ids"].tolist() == list(range(8)) * 2
    assert b["loss_mask"][7] == 0 and b["labels"][7] == 0                      # no target across the segment start
    assert b["labels"][8] == 209 and b["host_cu_seqlens"][:3].tolist() == [0, 8, 16]
    assert len(S.MLPerfPackedDataset(str(tmp_path), "validation")) == 1
