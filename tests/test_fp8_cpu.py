"""MXFP8 reference arithmetic (plain PyTorch): scale rule, block layout, round trip."""
import torch

from primus_b200.ops import fp8


def test_scale_is_smallest_power_of_two_that_avoids_saturation():
    amax = torch.tensor([448.0, 448.1, 1.0, 0.0, 3.5e-3, 2.0 ** 10 * 448])
    e = fp8._e8m0(amax).long() - 127
    assert e.tolist()[:3] == [0, 1, -8]
    assert fp8._e8m0(torch.tensor([0.0])).item() == 0
    nz = amax > 0
    assert ((amax[nz] / torch.exp2(e[nz].float())) <= 448.0).all()
    assert ((amax[nz] / torch.exp2(e[nz].float() - 1)) > 448.0).all()


def test_scale_block_layout_is_a_permutation_of_512_byte_blocks():
    R, C = 256, 384
    mn = torch.arange(R)[:, None].expand(R, C // 32)
    kb = torch.arange(C // 32)[None, :].expand(R, C // 32)
    off = fp8.sf_offsets(mn, kb, C // 128).reshape(-1)
    assert off.unique().numel() == R * C // 32 and off.max().item() == R * C // 32 - 1
    # row r, k-block j of a 128 x 128 block sits at (r % 32) * 16 + (r // 32) * 4 + j
    assert fp8.sf_offsets(torch.tensor(37), torch.tensor(2), 3).item() == 5 * 16 + 1 * 4 + 2
    assert fp8.sf_offsets(torch.tensor(128 + 37), torch.tensor(4 + 2), 3).item() == (3 + 1) * 512 + 5 * 16 + 4 + 2


def test_round_trip_error_and_cpu_linear():
    torch.manual_seed(0)
    x = (torch.randn(256, 256) * torch.exp(torch.randn(256, 1) * 2)).bfloat16()
    q = fp8.quantize_mxfp8_ref(x)
    for colwise, qq, sf in ((False, q.q_row, q.sf_row), (True, q.q_col, q.sf_col)):
        d = fp8.dequantize_mxfp8_ref(qq, sf, colwise)
        blocks = x.float().view(256, 8, 32) if not colwise else x.float().view(8, 32, 256)
        amax = blocks.abs().amax(-1 if not colwise else 1)
        bound = (amax / 448.0 * 2 * 16.0)  # half an ulp at the top binade (ulp 32) after rounding the scale up by < 2x
        err = (d - x.float()).abs().view_as(blocks).amax(-1 if not colwise else 1)
        assert (err <= bound + 1e-30).all()
    w = (torch.randn(128, 256) * 0.05).bfloat16()
    y = fp8.linear_mxfp8(x, w)
    ref = x.float() @ w.float().t()
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), ref.flatten(), dim=0)
    assert cos > 0.995


def test_tensorwise_recipe_uses_one_power_of_two_scale():
    """fp8_recipe tensorwise: every block carries the exponent of the tensor maximum, the dequantised values are the
    E4M3 rounding of x / 2^e, and both storage directions hold the same numbers."""
    torch.manual_seed(0)
    x = (torch.randn(256, 384) * 3).bfloat16()
    q = fp8.quantize_mxfp8_ref(x, True, True, tensorwise=True)
    e = fp8._e8m0(x.float().abs().amax().reshape(1)).item()
    assert (q.sf_row == e).all() and (q.sf_col == e).all()
    assert 448.0 / 2 < x.float().abs().max().item() / 2.0 ** (e - 127) <= 448.0
    want = (x.float() / 2.0 ** (e - 127)).to(torch.float8_e4m3fn).float() * 2.0 ** (e - 127)
    d_row = fp8.dequantize_mxfp8_ref(q.q_row, q.sf_row, False)
    d_col = fp8.dequantize_mxfp8_ref(q.q_col, q.sf_col, True)
    assert torch.equal(d_row, want) and torch.equal(d_col, want)
    # the module switch (set by the recipe) is the default of the quantiser
    from primus_b200.ops import gemm
    try:
        gemm.set_fp8_recipe("tensorwise")
        assert fp8.TENSORWISE and torch.equal(fp8.quantize_mxfp8(x, True, False).sf_row, q.sf_row)
    finally:
        gemm.set_fp8_recipe(None)
    assert not fp8.TENSORWISE
