"""Checkpoint: torch_dist directory layout, mcore key layout (QKV interleave round trip), bit-exact resume,
resharding to another TP size, finetune load."""
import json
import os

import torch

from primus_b200.engine import checkpoint as C
from primus_b200.engine.trainer import Trainer
from primus_b200.parallel import state as ps
from tests import dist_workers as W
from tests.mp_utils import run_ranks


def test_qkv_layout_roundtrip():
    hq, hkv, d, H = 8, 2, 4, 16
    w = torch.arange((hq + 2 * hkv) * d * H, dtype=torch.float32).view(-1, H)
    m = C.qkv_internal_to_mcore(w, hq, hkv, d)
    assert torch.equal(C.qkv_mcore_to_internal(m, hq, hkv, d), w)
    g = hq // hkv
    # group 0 of the interleaved layout: its g query heads, then k head 0, then v head 0
    assert torch.equal(m[: g * d], w[: g * d])
    assert torch.equal(m[g * d:(g + 1) * d], w[hq * d: hq * d + d])
    assert torch.equal(m[(g + 1) * d:(g + 2) * d], w[(hq + hkv) * d:(hq + hkv) * d + d])


def _dcp_metadata(d):
    from torch.distributed.checkpoint import FileSystemReader

    return FileSystemReader(d).read_metadata().state_dict_metadata


def _trainer(iters=6, **kw):
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=iters, **kw)
    return Trainer(mc, tc, device="cpu", log_fn=lambda s: None)


def test_save_layout_and_bitexact_resume(tmp_path):
    root = str(tmp_path / "ckpt")
    a = _trainer()
    first = a.train(3)
    d = a.save_checkpoint(root)
    rest_ref = a.train(3)
    assert os.path.basename(d) == "iter_0000003"
    assert open(os.path.join(root, C.TRACKER)).read().strip() == "3"
    assert {"common.pt", ".metadata", "__0_0.distcp"} <= set(os.listdir(d))
    common = torch.load(os.path.join(d, "common.pt"), weights_only=False)
    assert "args" in common and common["iteration"] == 3
    meta = _dcp_metadata(d)
    assert "decoder.layers.0.self_attention.linear_qkv.layer_norm_weight" in meta
    assert "decoder.layers.0.mlp.linear_fc1.weight" in meta and "embedding.word_embeddings.weight" in meta
    assert "output_layer.weight" in meta and "decoder.final_layernorm.weight" in meta
    b = _trainer()
    assert b.load_checkpoint(root) == 3
    rest = b.train(3)
    assert rest == rest_ref, (rest, rest_ref)  # same data stream, optimizer state and RNG: bit-identical losses
    assert len(first) == 3


def test_finetune_load_resets_iteration(tmp_path):
    root = str(tmp_path / "ckpt")
    a = _trainer()
    a.train(2)
    a.save_checkpoint(root)
    b = _trainer()
    assert C.load_checkpoint(b, root, finetune=True) == 0 and b.iteration == 0
    pa = dict(a.model.named_parameters())
    for n, p in b.model.named_parameters():
        assert torch.equal(p, pa[n])


def _reshard_worker(rank, world, root, outp, kw=None):
    ps.destroy_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=2, tp=2, sp=True, **(kw or dict(extra_mc=dict(add_qkv_bias=True))))
    ps.initialize_model_parallel(tp=2)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    tr.load_checkpoint(root)
    losses = tr.train(2)
    if rank == 0:
        json.dump(losses, open(outp, "w"))


def test_load_tp1_checkpoint_into_tp2(tmp_path):
    root = str(tmp_path / "ckpt")
    a = _trainer(iters=4, extra_mc=dict(add_qkv_bias=True))     # the q / k / v bias follows the weight's row layout
    a.tcfg.use_distributed_optimizer = True
    a.train(2)
    a.save_checkpoint(root)
    # the optimizer state is re-sliced for the new tensor-parallel layout: compare with the uninterrupted run
    ref = a.train(2)
    outp = str(tmp_path / "l.json")
    run_ranks(_reshard_worker, 2, "gloo", args=(root, outp), timeout=200)
    got = json.load(open(outp))
    for x, y in zip(got, ref):
        assert abs(x - y) <= 2e-3 * max(1.0, abs(y)), (got, ref)


def test_load_tp1_mla_checkpoint_into_tp2(tmp_path):
    """Multi-latent attention under tensor parallelism: head-split up-projections and output projection, replicated
    down-projections; weights and optimizer state of a tp = 1 checkpoint are re-sliced."""
    root = str(tmp_path / "ckpt")
    a = _trainer(iters=4, mla=True)
    a.tcfg.use_distributed_optimizer = True
    a.train(2)
    a.save_checkpoint(root)
    ref = a.train(2)
    outp = str(tmp_path / "l.json")
    run_ranks(_reshard_worker, 2, "gloo", args=(root, outp, dict(mla=True)), timeout=200)
    got = json.load(open(outp))
    for x, y in zip(got, ref):
        assert abs(x - y) <= 2e-3 * max(1.0, abs(y)), (got, ref)


def test_load_tp1_delta_net_checkpoint_into_tp2(tmp_path):
    """Head-split mixers keep several blocks in one fused weight: a tp = 1 checkpoint is re-tiled block by block (weights
    and optimizer state) for tp = 2."""
    kw = dict(layers=4, extra_mc=dict(
        model_type="kimi_k3", q_lora_rank=32, kv_lora_rank=24, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16,
        mla_use_output_gate=True, linear_attention_freq="[1, 0, 1, 0]", linear_num_key_heads=4, linear_num_value_heads=4,
        linear_key_head_dim=16, linear_value_head_dim=16, kda_chunk_size=16, attn_res_block_size=2))
    root = str(tmp_path / "ckpt")
    a = _trainer(iters=4, **kw)
    a.tcfg.use_distributed_optimizer = True
    a.train(2)
    a.save_checkpoint(root)
    ref = a.train(2)
    outp = str(tmp_path / "l.json")
    run_ranks(_reshard_worker, 2, "gloo", args=(root, outp, kw), timeout=200)
    got = json.load(open(outp))
    for x, y in zip(got, ref):
        assert abs(x - y) <= 2e-3 * max(1.0, abs(y)), (got, ref)


def _fsdp_ckpt_worker(rank, world, root, outp):
    import json as _json

    from primus_b200.engine.trainer import Trainer
    from primus_b200.parallel import state as _ps
    from tests import dist_workers as _W

    def make():
        _ps.destroy_model_parallel()
        _ps.initialize_model_parallel()
        mc, tc = _W.tiny_cfgs(seq=32, gbs=4, mbs=1, iters=4, fsdp=True)
        torch.manual_seed(11)
        return Trainer(mc, tc, device="cpu", log_fn=lambda s: None)

    a = make()
    a.train(2)
    a.save_checkpoint(root)
    ref = a.train(2)
    b = make()
    assert b.load_checkpoint(root) == 2
    got = b.train(2)
    if rank == 0:
        with open(outp, "w") as f:
            _json.dump({"ref": ref[-2:], "got": got[-2:]}, f)


def test_fsdp2_checkpoint_resume(tmp_path):
    """use_torch_fsdp2: parameters are saved whole, the Adam moments as per-rank shards; a fresh trainer continues
    exactly where the saved one stood."""
    root, outp = str(tmp_path / "ckpt"), str(tmp_path / "l.json")
    run_ranks(_fsdp_ckpt_worker, 2, "gloo", args=(root, outp), timeout=240)
    r = json.load(open(outp))
    assert r["ref"] == r["got"], r
    meta = _dcp_metadata(os.path.join(root, "iter_0000002"))
    emb = meta["embedding.word_embeddings.weight"]
    assert len(emb.chunks) == 2 and tuple(emb.size) == (512, 64)      # one chunk per data-parallel rank


def test_checkpoint_is_readable_by_plain_dcp(tmp_path):
    """The files are stock torch.distributed.checkpoint files: ``dcp.load`` fills plain tensors of the global shapes
    without any code of this package, and the values are the model's (QKV rows in the Megatron-core interleave)."""
    import torch.distributed.checkpoint as dcp

    root = str(tmp_path / "ckpt")
    a = _trainer()
    a.train(1)
    d = a.save_checkpoint(root)
    md = _dcp_metadata(d)
    keys = ["decoder.layers.1.self_attention.linear_qkv.weight", "decoder.layers.0.mlp.linear_fc2.weight",
            "optimizer.state.exp_avg.decoder.layers.0.mlp.linear_fc2.weight"]
    sd = {k: torch.zeros(tuple(md[k].size), dtype=md[k].properties.dtype) for k in keys}
    dcp.load(sd, checkpoint_id=d, no_dist=True)
    params = dict(a.model.named_parameters())
    cfg = a.mcfg
    qkv = params["decoder.layers.1.self_attention.linear_qkv.weight"]
    assert torch.equal(sd[keys[0]], C.qkv_internal_to_mcore(qkv.detach(), cfg.num_attention_heads, cfg.num_query_groups,
                                                            cfg.kv_channels))
    assert torch.equal(sd[keys[1]], params["decoder.layers.0.mlp.linear_fc2.weight"].detach())
    assert sd[keys[2]].abs().sum() > 0


def test_async_save_and_torch_format(tmp_path):
    root = str(tmp_path / "a")
    a = _trainer()
    a.tcfg.async_save = True
    a.train(2)
    a.save_checkpoint(root)
    ref = a.train(2)                       # training continues while the files are written
    C.finalize_async_save()
    b = _trainer()
    assert b.load_checkpoint(root) == 2 and b.train(2) == ref
    # legacy per-rank pickles, found by auto-detection
    root2 = str(tmp_path / "t")
    c = _trainer()
    c.tcfg.ckpt_format = "torch"
    c.train(2)
    d = c.save_checkpoint(root2)
    ref2 = c.train(2)
    assert os.path.exists(os.path.join(d, "mp_rank_00", "model_optim_rng.pt"))
    e = _trainer()
    e.tcfg.auto_detect_ckpt_format = True
    assert e.load_checkpoint(root2) == 2 and e.train(2) == ref2


def test_strictness_and_missing_optimizer_state(tmp_path):
    import pytest

    root = str(tmp_path / "ckpt")
    a = _trainer()
    a.tcfg.no_save_optim = True
    a.train(1)
    a.save_checkpoint(root)
    logs = []
    b = _trainer()
    b.log = logs.append
    assert b.load_checkpoint(root) == 1            # weights load; the reset of the optimizer is said out loud
    assert any("without optimizer state" in l for l in logs)
    # a model with an extra layer: its tensors are missing from the checkpoint
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=2, layers=6)
    c = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    with pytest.raises(KeyError, match="lacks"):
        c.load_checkpoint(root)
    c.tcfg.dist_ckpt_strictness = "log_all"
    c.tcfg.no_load_optim = True
    logs2 = []
    c.log = logs2.append
    assert c.load_checkpoint(root) == 1 and any("missing keys" in l for l in logs2)


def _dp_worker(rank, world, root, outp, phase):
    ps.destroy_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=8, mbs=1, iters=4)
    tc.ckpt_fully_parallel_load = True
    ps.initialize_model_parallel()
    torch.manual_seed(5)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    if phase == "save":
        tr.train(2)
        tr.save_checkpoint(root)
        rest = tr.train(2)
    else:
        assert tr.load_checkpoint(root) == 2
        rest = tr.train(2)
    if rank == 0:
        json.dump(rest, open(outp, "w"))


def test_resume_with_another_data_parallel_size(tmp_path):
    """Saved on 2 data-parallel ranks (each holds half of every ZeRO-1 shard), resumed on 4 and on 1: the optimizer
    state is re-sliced from the chunk metadata and the next losses agree with the uninterrupted run."""
    root = str(tmp_path / "ckpt")
    run_ranks(_dp_worker, 2, "gloo", args=(root, str(tmp_path / "ref.json"), "save"), timeout=240)
    ref = json.load(open(tmp_path / "ref.json"))
    run_ranks(_dp_worker, 4, "gloo", args=(root, str(tmp_path / "dp4.json"), "load"), timeout=240)
    got4 = json.load(open(tmp_path / "dp4.json"))
    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=8, mbs=1, iters=4)
    one = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    assert one.load_checkpoint(root) == 2
    got1 = one.train(2)
    for got in (got4, got1):
        for x, y in zip(got, ref):
            assert abs(x - y) <= 1e-5 * max(1.0, abs(y)), (got, ref)


def test_non_persistent_checkpoints_keep_only_the_newest_and_win_when_newer(tmp_path):
    root = str(tmp_path / "ckpt")
    a = _trainer(iters=7, extra_tc=dict(save=root, save_interval=4, non_persistent_ckpt_type="global",
                                        non_persistent_save_interval=1))
    ref = a.train(7)
    np_root = os.path.join(root, "non_persistent")
    assert sorted(n for n in os.listdir(np_root) if n.startswith("iter_")) == ["iter_0000007"]
    assert os.path.isdir(os.path.join(root, "iter_0000004")) and C.latest_iteration(root) == 4
    # a fresh trainer resumes from the newer, non-persistent state (iteration 7), not from the persistent one (4)
    logs = []
    b = _trainer(iters=9, extra_tc=dict(save=root, non_persistent_ckpt_type="global"))
    b.log = logs.append
    assert b.load_checkpoint(root) == 7 and any("non-persistent" in l for l in logs)
    c = _trainer(iters=9, extra_tc=dict(save=root))
    assert c.load_checkpoint(root) == 4
    more_ref = a.train(2)
    assert b.train(2) == more_ref and len(ref) == 7


def test_checkpoint_format_conversion_run(tmp_path):
    """``ckpt_convert_format``: a run that loads a torch_dist checkpoint, writes it in the legacy torch layout and leaves;
    training from the converted checkpoint continues like from the original."""
    from primus_b200.engine.pretrain import PretrainTrainer

    a = _trainer()
    a.train(2)
    a.save_checkpoint(str(tmp_path / "dist"))
    ref = a.train(2)
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=6)
    params = dict(vars(mc), **vars(tc))
    params.update(load=str(tmp_path / "dist"), ckpt_convert_format="torch", ckpt_convert_save=str(tmp_path / "legacy"),
                  mock_data=True)
    ps.destroy_model_parallel()
    t = PretrainTrainer.__new__(PretrainTrainer)
    t.params, t.runtime_state, t.world_size, t.local_rank = params, None, 1, 0
    t.init()
    t.train()
    assert t.engine.iteration == 2 and os.path.isdir(tmp_path / "legacy" / "iter_0000002" / "mp_rank_00")
    b = _trainer()
    b.tcfg.auto_detect_ckpt_format = True
    assert b.load_checkpoint(str(tmp_path / "legacy")) == 2
    got = b.train(2)
    assert all(abs(x - y) < 1e-5 for x, y in zip(got, ref)), (got, ref)
