"""A device-side wait that runs out must report through the status word and leave the context usable.

The flag lives in this GPU's own memory and nothing ever sets it, so no peer and no second kernel is involved: the wait
kernel spins for a small, fixed number of clock cycles (about a millisecond), records ``PB_ERR_TIMEOUT_FLAG`` and returns.
"""
import pytest
import torch

from primus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_context_survives():
    _lib.require()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    st = _lib.status_word(dev)
    st.zero_()
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.call("flag_wait", flag, _lib.i32(1), st, 2_000_000)      # ~1 ms at B200 clocks
    torch.cuda.synchronize()
    with pytest.raises(_lib.NativeLibraryError, match="status 4"):
        _lib.check_status(dev)
    # the status word is cleared by the check and the next kernels run normally
    _lib.check_status(dev)
    _lib.call("flag_set", flag, _lib.i32(1))
    _lib.call("flag_wait", flag, _lib.i32(1), st, 2_000_000)      # satisfied at once
    torch.cuda.synchronize()
    _lib.check_status(dev)
    a = torch.randn(256, 256, device=dev).bfloat16()
    from primus_b200.ops import gemm

    out = gemm.gemm(a, a)
    ref = a.float() @ a.float().t()
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=0.5)
