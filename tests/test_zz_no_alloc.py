"""The allocation-free RMSNorm-backward entry point (``pb_rmsnorm_bwd_noalloc``).

Some users of the library cannot allocate device memory where they call it (a host application that
owns all allocations, a fixed arena, a latency-critical loop), so this entry point keeps its scratch in
a fixed array inside the library.  The test calls it through its exported C symbol twice in a row and
compares with the regular entry point, which takes caller-provided scratch.  The file is named so that
pytest collects it last.
"""
import ctypes

import pytest
import torch

from primus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, dy, x, w, rstd, dres, dx, dw, accumulate):
    fn = lib.pb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    vp = ctypes.c_void_p
    rows, H = x.shape
    return fn(vp(dy.data_ptr()), vp(x.data_ptr()), vp(w.data_ptr()), vp(rstd.data_ptr()),
              vp(dres.data_ptr() if dres is not None else 0), vp(dx.data_ptr()), vp(dw.data_ptr()),
              ctypes.c_long(rows), ctypes.c_int(H), ctypes.c_long(x.stride(0)), ctypes.c_long(dy.stride(0)),
              ctypes.c_int(int(accumulate)), vp(torch.cuda.current_stream().cuda_stream))


def _reference(dy, x, w, rstd, dres):
    rows, H = x.shape
    dx = torch.empty_like(x)
    dw = torch.zeros(H, dtype=torch.float32, device=x.device)
    P = _lib.call_ret("rmsnorm_bwd_num_partials", rows)
    scratch = torch.empty(P * H, dtype=torch.float32, device=x.device)
    _lib.call("rmsnorm_bwd", dy, x, w, rstd, dres, dx, dw, scratch, rows, H, x.stride(0), dy.stride(0), 0)
    return dx, dw


# (300, 8192): the documented maximum width, with more rows than the 296 partial rows of the built-in scratch
@pytest.mark.parametrize("rows,H,with_res", [(1000, 4096, True), (77, 512, False), (300, 8192, True)])
def test_noalloc_matches_regular_entry_point_twice(rows, H, with_res):
    lib = _lib.require()
    g = torch.Generator(device="cuda").manual_seed(rows + H)
    results = []
    for call in range(2):  # two calls in a row share the built-in scratch
        x = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
        dy = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
        dres = torch.randn(rows, H, device="cuda", generator=g).bfloat16() if with_res else None
        w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        dx_ref, dw_ref = _reference(dy, x, w, rstd, dres)
        dx = torch.empty_like(x)
        dw = torch.zeros(H, dtype=torch.float32, device="cuda")
        rc = _call_noalloc(lib, dy, x, w, rstd, dres, dx, dw, accumulate=False)
        assert rc == 0, f"pb_rmsnorm_bwd_noalloc returned {rc}"
        torch.cuda.synchronize()
        err_dx = (dx.float() - dx_ref.float()).abs().max().item()
        assert err_dx <= 2e-2 + 2e-2 * dx_ref.float().abs().max().item(), f"call {call}: dx err {err_dx}"
        err_dw = (dw - dw_ref).abs().max().item()
        # both entry points run the same kernels in the same order: a dropped or stale partial row would show
        assert err_dw <= 1e-3 * dw_ref.abs().max().item() + 1e-5, f"call {call}: dw err {err_dw}"
        results.append((dx, dw))
    # accumulate mode adds onto the existing weight gradient
    dx2 = torch.empty_like(x)
    dw2 = results[-1][1].clone()
    assert _call_noalloc(lib, dy, x, w, rstd, dres, dx2, dw2, accumulate=True) == 0
    torch.cuda.synchronize()
    assert (dw2 - 2 * results[-1][1]).abs().max().item() <= 1e-3 + 1e-3 * dw2.abs().max().item()


def test_noalloc_rejects_oversized_rows():
    lib = _lib.require()
    H = 8192 + 8
    x = torch.zeros(4, H, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(H, device="cuda")
    rstd = torch.ones(4, device="cuda")
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rc = _call_noalloc(lib, x, x, w, rstd, None, torch.empty_like(x), dw, False)
    assert rc == -10  # PB_NOALLOC_ERR_TOO_LARGE: nothing was launched
