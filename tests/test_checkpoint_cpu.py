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
    meta = json.load(open(os.path.join(d, ".metadata")))["tensors"]
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


def _reshard_worker(rank, world, root, outp):
    ps.destroy_model_parallel()
    mc, tc = W.tiny_cfgs(seq=32, gbs=4, mbs=2, iters=2, tp=2, sp=True)
    ps.initialize_model_parallel(tp=2)
    tr = Trainer(mc, tc, device="cpu", log_fn=lambda s: None)
    tr.load_checkpoint(root)
    losses = tr.train(2)
    if rank == 0:
        json.dump(losses, open(outp, "w"))


def test_load_tp1_checkpoint_into_tp2(tmp_path):
    root = str(tmp_path / "ckpt")
    a = _trainer(iters=4)
    a.tcfg.use_distributed_optimizer = True
    a.train(2)
    a.save_checkpoint(root)
    # continue without optimizer state on the reference too (layout change drops the moments)
    b = _trainer(iters=4)
    C.load_checkpoint(b, root, load_optim=False)
    ref = b.train(2)
    outp = str(tmp_path / "l.json")
    run_ranks(_reshard_worker, 2, "gloo", args=(root, outp), timeout=200)
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
    meta = json.load(open(os.path.join(root, "iter_0000002", ".metadata")))["tensors"]
    assert "embedding.word_embeddings.weight" in meta and len(meta["embedding.word_embeddings.weight"]) == 1
