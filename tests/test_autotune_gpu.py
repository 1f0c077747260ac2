"""Online tile tuning on the device: candidates are timed, the winner is used, results do not change."""
import pytest
import torch

from primus_b200.ops import _lib, autotune, gemm

pytestmark = pytest.mark.gpu


def test_online_tuning_picks_a_candidate_and_keeps_results_bitwise():
    torch.manual_seed(0)
    a = torch.randn(512, 1024, device="cuda").bfloat16()
    b = torch.randn(768, 1024, device="cuda").bfloat16()
    autotune.clear()
    ref = gemm.gemm(a, b)
    try:
        autotune.set_online(True)
        out = gemm.gemm(a, b)
        key = autotune.make_key("bf16", 512, 768, 1024, False, False, 0)
        entry = autotune.table()[key]
        assert entry.get("block_n") in (128, 256) and entry["time_us"] > 0 and len(entry["candidates_us"]) == 2
        assert torch.equal(out, ref)            # the tile width does not change the accumulation order over K
        gemm.set_fp8_recipe("mxfp8")
        out8 = gemm.gemm(a, b)
        key8 = autotune.make_key("mxfp8", 512, 768, 1024, False, False, 0)
        assert key8 in autotune.table()
        assert torch.equal(out8, gemm.gemm(a, b))
        torch.cuda.synchronize()
        _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)
        autotune.set_online(False)
        autotune.clear()
