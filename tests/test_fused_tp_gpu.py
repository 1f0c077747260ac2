"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels vs the NCCL + GEMM composition and vs an fp32 evaluation of
the same products (2 GPUs)."""
import pytest
import torch

from tests.mp_utils import run_ranks

pytestmark = pytest.mark.gpu


def _worker(rank, world, shapes):
    import torch.distributed as dist

    from primus_b200.ops import _lib
    from primus_b200.parallel import fused_tp

    group = dist.group.WORLD
    torch.manual_seed(1234 + rank)
    torch.backends.cuda.matmul.allow_tf32 = False
    for (T, N, K, b_mn) in shapes:
        Tl = T // world
        for it in range(3):  # several epochs through the same workspace
            x_shard = torch.randn(Tl, K, device="cuda").bfloat16()
            w = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).bfloat16()
            out, gathered = fused_tp.ag_gemm(x_shard, w, group, b_mn=b_mn, fused=True)
            ref, gref = fused_tp.ag_gemm(x_shard, w, group, b_mn=b_mn, fused=False)
            torch.cuda.synchronize()
            _lib.check_status()
            assert torch.equal(gathered, gref), f"gathered activations differ (T={T} it={it})"
            err = (out.float() - ref.float()).abs().max().item()
            assert err <= 2e-2 * ref.float().abs().max().item() + 1e-3, f"ag_gemm err {err}"
            # fp32 evaluation of the same product from the gathered operands (torch matmul in fp32, no TF32)
            wf = w.float() if b_mn else w.float().t()
            xs = [torch.empty_like(x_shard) for _ in range(world)]
            dist.all_gather(xs, x_shard, group=group)
            ref32 = torch.cat(xs).float() @ wf
            err32 = (out.float() - ref32).abs().max().item()
            assert err32 <= 1e-2 * ref32.abs().max().item() + 1e-3, f"ag_gemm vs fp32: {err32}"
            x = torch.randn(T, K, device="cuda").bfloat16()
            out2 = fused_tp.gemm_rs(x, w, group, b_mn=b_mn, fused=True)
            ref2 = fused_tp.gemm_rs(x, w, group, b_mn=b_mn, fused=False)
            torch.cuda.synchronize()
            _lib.check_status()
            err2 = (out2.float() - ref2.float()).abs().max().item()
            assert err2 <= 3e-2 * ref2.float().abs().max().item() + 1e-2, f"gemm_rs err {err2}"
            # fp32: every rank's partial product of its own (x, w), summed over the ranks, this rank's rows
            part = (x.float() @ wf)
            dist.all_reduce(part, group=group)
            ref32 = part[rank * Tl:(rank + 1) * Tl]
            err32 = (out2.float() - ref32).abs().max().item()
            assert err32 <= 1.5e-2 * ref32.abs().max().item() + 1e-2, f"gemm_rs vs fp32: {err32}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_matches_nccl_composition():
    shapes = [(512, 256, 128, False), (2048, 1280, 1024, False), (1024, 768, 512, True)]
    run_ranks(_worker, 2, "nccl", args=(shapes,), timeout=240)


@pytest.mark.parametrize("world", [4, 8])
def test_fused_tp_with_several_remote_sources(world):
    """More than one remote source: the copy CTAs add the partial products of all remote ranks per piece."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    shapes = [(2048, 1280, 1024, False), (1024, 768, 512, True)]
    run_ranks(_worker, world, "nccl", args=(shapes,), timeout=240)


def _repeat_worker(rank, world, shapes):
    import os

    import torch.distributed as dist

    from primus_b200.ops import _lib
    from primus_b200.parallel import fused_tp

    group = dist.group.WORLD
    torch.manual_seed(4321 + rank)
    os.environ["PRIMUS_B200_RS_TEST_REPEAT"] = "1"
    try:
        for (T, N, K) in shapes:
            Tl = T // world
            for it in range(3):
                x = torch.randn(T, K, device="cuda").bfloat16()
                w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
                out = fused_tp.gemm_rs(x, w, group, fused=True)
                torch.cuda.synchronize()
                _lib.check_status()
                ref = fused_tp.gemm_rs(x, w, group, fused=False).float()
                own = (x[rank * Tl:(rank + 1) * Tl].float() @ w.float().t())
                want = 2.0 * ref - own          # own + 2 x (the peer's partial product)
                err = (out.float() - want).abs().max().item()
                assert err <= 3e-2 * want.abs().max().item() + 2e-2, f"T={T} it={it}: err {err}"
    finally:
        os.environ.pop("PRIMUS_B200_RS_TEST_REPEAT", None)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_reduce_scatter_accumulates_over_passes():
    """The pass structure tensor-parallel sizes above 3 use (sources added in arrival order, the accumulator re-read
    between passes), driven on 2 GPUs by the kernel's test hook: the peer's partial product is added in two passes."""
    run_ranks(_repeat_worker, 2, "nccl", args=([(2048, 1280, 1024), (1024, 768, 512)],), timeout=240)
