"""The plumbing benchmark configuration, exactly as specified: a tiny Llama-style decoder (4 layers, hidden 256, 4 query /
2 KV heads of 64, SwiGLU FFN 688, RMSNorm eps 1e-5, RoPE theta 10000, vocab 32000, untied embeddings, N(0, 0.02) init),
fp32, data parallel over 2 gloo ranks, 10 AdamW steps (lr 3e-4, betas 0.9 / 0.95, weight decay 0.1), sequence 512,
micro-batch 2, global batch 8, uniform token ids from seed 1234 with labels shifted by one.

The reference's Megatron backend cannot run here, so the trajectory is checked twice: against an independent
restatement of the model and optimizer in plain ``torch.nn`` / ``torch.optim`` code (same initial weights, same batches),
and against the committed numbers of that restatement (``tests/golden/baseline_config1_losses.json``)."""
import json
import math
import os

import torch
import torch.nn.functional as F

from tests.mp_utils import run_ranks

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "baseline_config1_losses.json")
H, L, HQ, HKV, D, FFN, V, SEQ, MBS, GBS, STEPS = 256, 4, 4, 2, 64, 688, 32000, 512, 2, 8, 10


def _cfgs():
    from primus_b200.engine.trainer import TrainConfig
    from primus_b200.models.config import TransformerConfig

    mc = TransformerConfig(num_layers=L, hidden_size=H, ffn_hidden_size=FFN, num_attention_heads=HQ, num_query_groups=HKV,
                           kv_channels=D, vocab_size=V, params_dtype="fp32", norm_epsilon=1e-5, rotary_base=10000.0,
                           init_method_std=0.02, untie_embeddings_and_output_weights=True,
                           make_vocab_size_divisible_by=128)
    tc = TrainConfig(micro_batch_size=MBS, global_batch_size=GBS, seq_length=SEQ, train_iters=STEPS, lr=3e-4,
                     lr_decay_style="constant", weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95, clip_grad=1.0,
                     seed=1234, data_seed=1234, log_interval=1)
    return mc, tc


class PlainLlama(torch.nn.Module):
    """Independent restatement: standard PyTorch ops only, weights copied from the engine's state dict."""

    def __init__(self, sd):
        super().__init__()
        self.p = torch.nn.ParameterDict({k.replace(".", "/"): torch.nn.Parameter(v.clone().float()) for k, v in sd.items()})

    def w(self, name):
        return self.p[name.replace(".", "/")]

    @staticmethod
    def rms(x, w, eps=1e-5):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    @staticmethod
    def rope(x, theta=10000.0):
        b, s, h, d = x.shape
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        ang = torch.arange(s, dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[None, :, None, :], torch.cat([ang.sin(), ang.sin()], -1)[None, :, None, :]
        rot = torch.cat([-x[..., d // 2:], x[..., : d // 2]], -1)
        return x * cos + rot * sin

    def forward(self, tokens, labels):
        b, s = tokens.shape
        x = self.w("embedding.word_embeddings.weight")[tokens]
        for i in range(L):
            pre = f"decoder.layers.{i}."
            y = self.rms(x, self.w(pre + "self_attention.linear_qkv.layer_norm_weight"))
            qkv = y @ self.w(pre + "self_attention.linear_qkv.weight").t()
            q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], -1)
            q = self.rope(q.view(b, s, HQ, D)).transpose(1, 2)
            k = self.rope(k.view(b, s, HKV, D)).transpose(1, 2).repeat_interleave(HQ // HKV, 1)
            v = v.view(b, s, HKV, D).transpose(1, 2).repeat_interleave(HQ // HKV, 1)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, HQ * D)
            x = x + a @ self.w(pre + "self_attention.linear_proj.weight").t()
            y = self.rms(x, self.w(pre + "mlp.linear_fc1.layer_norm_weight"))
            gu = y @ self.w(pre + "mlp.linear_fc1.weight").t()
            g, u = gu.chunk(2, -1)
            x = x + (F.silu(g) * u) @ self.w(pre + "mlp.linear_fc2.weight").t()
        x = self.rms(x, self.w("decoder.final_layernorm.weight"))
        logits = x @ self.w("output_layer.weight").t()
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))


def _plain_trajectory():
    from primus_b200.engine.data import MicroBatchSampler, MockGPTDataset
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = _cfgs()
    torch.manual_seed(tc.seed)
    sd = {k: v.detach().clone() for k, v in GPTModel(mc, "cpu").state_dict().items()}
    ps.destroy_model_parallel()
    m = PlainLlama(sd)
    decay = [p for p in m.parameters() if p.dim() >= 2]
    no_decay = [p for p in m.parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=3e-4, betas=(0.9, 0.95), eps=1e-8)
    ds = MockGPTDataset(V, SEQ, 1234)
    losses, idx = [], 0
    for _ in range(STEPS):
        opt.zero_grad()
        total = 0.0
        for _mb in range(GBS // MBS):
            samples = [ds[idx + j] for j in range(MBS)]
            idx += MBS
            tok = torch.stack([torch.as_tensor(s_["tokens"]) for s_ in samples]).long()
            lab = torch.stack([torch.as_tensor(s_["labels"]) for s_ in samples]).long()
            loss = m(tok, lab) / (GBS // MBS)
            loss.backward()
            total += float(loss.detach())
        torch.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
        losses.append(total)
    return sd, losses


def _worker(rank, world, sd_path, out_path):
    from primus_b200.engine import checkpoint as C
    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = _cfgs()
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    sd = torch.load(sd_path)
    for n, p in tr.model.named_parameters():
        p.data.copy_(sd[n])
    C._refresh_master_weights(tr)
    losses = tr.train()
    if rank == 0:
        json.dump(losses, open(out_path, "w"))


def test_ten_step_trajectory_dp2_matches_independent_restatement(tmp_path):
    sd, ref = _plain_trajectory()
    if os.environ.get("PRIMUS_WRITE_GOLDEN") == "1":
        json.dump({"losses": ref}, open(GOLDEN, "w"), indent=1)
    sd_path, out = str(tmp_path / "sd.pt"), str(tmp_path / "l.json")
    torch.save(sd, sd_path)
    run_ranks(_worker, 2, "gloo", args=(sd_path, out), timeout=600)
    got = json.load(open(out))
    assert len(got) == STEPS == len(ref)
    assert abs(got[0] - math.log(V)) < 0.1                     # random init: loss ~ ln(vocab)
    for a, b in zip(got, ref):
        assert abs(a - b) <= 2e-4 * b, (got, ref)
    golden = json.load(open(GOLDEN))["losses"]
    for a, b in zip(got, golden):
        assert abs(a - b) <= 5e-4 * b, (got, golden)
