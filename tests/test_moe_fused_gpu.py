"""Fused expert-parallel dispatch+GEMM / GEMM+combine kernels (csrc/moe_fused.cu).

* 1 GPU (ep = 1): the device-side routing plan against a plain PyTorch restatement, and the fused MoE layer
  against the un-fused local path (same weights): output and gradients.
* 2 GPUs (ep = 2): fused path against the NCCL all-to-all path of the same layer on every rank.
"""
import copy

import pytest
import torch

from tests.mp_utils import run_ranks

pytestmark = pytest.mark.gpu


def _moe_cfg(**kw):
    from primus_b200.models.config import TransformerConfig

    base = dict(num_layers=1, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2, vocab_size=512,
                params_dtype="bf16", num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=128, moe_layer_freq=[1],
                moe_aux_loss_coeff=0.0, seq_length=384)
    base.update(kw)
    return TransformerConfig(**base)


def _plan_reference(idx, ep, rank_counts_all, rank, E, rows_cap):
    """Destination row of every copy of `rank`, from the [ep, E] count table (plain PyTorch)."""
    e_local = E // ep
    tot = rank_counts_all.sum(0)
    padded = (tot + 127) // 128 * 128
    row_start = torch.zeros(E, dtype=torch.long)
    for d in range(ep):
        acc = 0
        for le in range(e_local):
            row_start[d * e_local + le] = acc
            acc += int(padded[d * e_local + le])
    base_me = rank_counts_all[:rank].sum(0)
    flat = idx.reshape(-1).cpu().long()
    rows = torch.empty_like(flat)
    seen = torch.zeros(E, dtype=torch.long)
    for i, e in enumerate(flat.tolist()):
        rows[i] = row_start[e] + base_me[e] + seen[e]
        seen[e] += 1
    return rows, flat // e_local


def test_plan_matches_reference_single_rank():
    from primus_b200.ops import _lib
    from primus_b200.parallel import fused_ep

    T, k, E, H = 384, 2, 8, 256
    torch.manual_seed(3)
    ws = fused_ep.FusedEP(None, T, k, E, H)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
    probs = torch.rand(T, k, device="cuda")
    plan = ws.plan(idx, probs).finalize()
    torch.cuda.synchronize()
    _lib.check_status()
    counts = torch.bincount(idx.reshape(-1).cpu(), minlength=E).view(1, E)
    rows, dest = _plan_reference(idx, 1, counts, 0, E, ws.rows_cap)
    pull = plan.pull_src.cpu().long()
    inv = plan.inv_order.cpu().long().reshape(-1)
    assert torch.equal(pull[inv] & 0xffffff, rows)
    assert torch.equal(pull[inv] >> 24, dest)
    src = plan.src_map.cpu().long()
    tok = torch.arange(T).repeat_interleave(k)
    assert torch.equal(src[rows] & 0xffffff, tok)
    assert int((src >= 0).sum()) == T * k
    assert torch.allclose(plan.probs_perm.cpu()[rows], probs.reshape(-1).cpu())
    assert torch.equal(plan.tok_sorted.cpu().long()[inv], tok)
    assert torch.equal(plan.sched.counts.cpu().long(), counts[0])


def _layer_pair(cfg, seed=0):
    from primus_b200.models.gpt import GPTModel

    torch.manual_seed(seed)
    model = GPTModel(cfg, device="cuda")
    fused_model = copy.deepcopy(model)
    for m in fused_model.modules():
        if hasattr(m, "cfg"):
            m.cfg = copy.copy(m.cfg)
            m.cfg.use_turbo_mega_moe = True
    return model, fused_model


def _compare_models(model, fused_model, tokens, labels, tol=3e-2):
    from primus_b200.ops import _lib

    outs = []
    for m in (model, fused_model):
        loss = m(tokens, labels).mean()
        loss.backward()
        outs.append(loss.item())
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(outs[0] - outs[1]) <= 2e-3 * max(1.0, abs(outs[0])), outs
    ref = dict(model.named_parameters())
    for name, p in fused_model.named_parameters():
        g, r = p.grad, ref[name].grad
        assert (g is None) == (r is None), name
        if g is None:
            continue
        err = (g.float() - r.float()).abs().max().item()
        assert err <= tol * r.float().abs().max().item() + 1e-4, f"{name}: {err} vs {r.float().abs().max().item()}"


def _fp32_cpu_reference(cfg, model, tokens, labels):
    """Loss and gradients of the same weights evaluated by the plain PyTorch path in fp32 on the CPU."""
    import dataclasses

    from primus_b200.models.gpt import GPTModel

    cfg32 = dataclasses.replace(cfg, params_dtype="fp32", use_turbo_mega_moe=False)
    ref = GPTModel(cfg32, device="cpu")
    ref.load_state_dict({k: v.detach().float().cpu() for k, v in model.state_dict().items()})
    loss = ref(tokens.cpu(), labels.cpu()).mean()
    loss.backward()
    return loss.item(), {n: p.grad for n, p in ref.named_parameters()}


def test_fused_layer_matches_fp32_reference_single_rank():
    """The fused dispatch + GEMM / GEMM + combine path against an fp32 evaluation of the same layer (not only against
    this package's own un-fused composition): loss within bf16 rounding, every gradient highly correlated."""
    from primus_b200.ops import _lib

    cfg = _moe_cfg(moe_aux_loss_coeff=1e-2)
    _, fused_model = _layer_pair(cfg)
    tokens = torch.randint(0, 512, (1, cfg.seq_length), device="cuda")
    labels = torch.randint(0, 512, (1, cfg.seq_length), device="cuda")
    loss = fused_model(tokens, labels).mean()
    loss.backward()
    torch.cuda.synchronize()
    _lib.check_status()
    ref_loss, ref_grads = _fp32_cpu_reference(cfg, fused_model, tokens, labels)
    assert abs(loss.item() - ref_loss) <= 5e-3 * abs(ref_loss), (loss.item(), ref_loss)
    for name, p in fused_model.named_parameters():
        g, r = p.grad, ref_grads[name]
        if g is None or r is None or r.abs().max() == 0:
            continue
        cos = torch.nn.functional.cosine_similarity(g.float().cpu().flatten(), r.flatten(), dim=0).item()
        assert cos >= 0.98, (name, cos)


@pytest.mark.parametrize("score", ["softmax", "sigmoid"])
def test_fused_layer_matches_local_path_single_rank(score):
    cfg = _moe_cfg(moe_router_score_function=score, moe_aux_loss_coeff=1e-2)
    model, fused_model = _layer_pair(cfg)
    tokens = torch.randint(0, 512, (1, cfg.seq_length), device="cuda")
    labels = torch.randint(0, 512, (1, cfg.seq_length), device="cuda")
    for _ in range(2):  # second pass reuses the workspace (epochs, counters)
        for m in (model, fused_model):
            m.zero_grad(set_to_none=True)
        _compare_models(model, fused_model, tokens, labels)


def _ep_worker(rank, world):
    import torch.distributed as dist

    from primus_b200.models.gpt import GPTModel
    from primus_b200.ops import _lib
    from primus_b200.parallel import state as ps

    ps.initialize_model_parallel(ep=world)
    cfg = _moe_cfg(num_experts=8, moe_router_topk=2, hidden_size=256, seq_length=512, moe_aux_loss_coeff=1e-2,
                   expert_model_parallel_size=world)
    torch.manual_seed(11)
    model = GPTModel(cfg, device="cuda")
    fused_model = copy.deepcopy(model)
    for m in fused_model.modules():
        if hasattr(m, "cfg"):
            m.cfg = copy.copy(m.cfg)
            m.cfg.use_turbo_mega_moe = True
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    for it in range(3):
        tokens = torch.randint(0, 512, (1, cfg.seq_length), device="cuda", generator=g)
        labels = torch.randint(0, 512, (1, cfg.seq_length), device="cuda", generator=g)
        for m in (model, fused_model):
            m.zero_grad(set_to_none=True)
        _compare_models(model, fused_model, tokens, labels)
    dist.barrier()
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ep_matches_nccl_all_to_all():
    run_ranks(_ep_worker, 2, "nccl", timeout=300)
