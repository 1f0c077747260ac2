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


def test_blockwise_recipe_scales_vectors_of_128_and_weight_tiles():
    """fp8_recipe blockwise: an activation takes one exponent per 1 x 128 vector along the reduced dimension (row
    direction: along columns; column direction: along rows), a weight one per 128 x 128 tile; the four 32-blocks a
    vector covers carry the same exponent."""
    torch.manual_seed(0)
    x = (torch.randn(256, 384) * torch.exp(torch.randn(256, 1) * 2)).bfloat16()
    q = fp8.quantize_mxfp8_ref(x, True, True, scaling="blockwise")
    R, C = x.shape
    r = torch.arange(R)[:, None].expand(R, C // 32)
    kb = torch.arange(C // 32)[None, :].expand(R, C // 32)
    e_row = q.sf_row[fp8.sf_offsets(r, kb, C // 128).reshape(-1)].view(R, C // 128, 4)
    assert (e_row == e_row[..., :1]).all()
    want = fp8._e8m0(x.float().abs().view(R, C // 128, 128).amax(-1))
    assert torch.equal(e_row[..., 0].int(), want)
    d = fp8.dequantize_mxfp8_ref(q.q_row, q.sf_row, False)
    assert ((d - x.float()).abs() <= x.float().abs().view(R, C // 128, 128).amax(-1).repeat_interleave(128, 1) * 0.0626 / 1.0).all()
    # column direction: vectors of 128 rows
    c = torch.arange(C)[None, :].expand(R // 32, C)
    rb = torch.arange(R // 32)[:, None].expand(R // 32, C)
    e_col = q.sf_col[fp8.sf_offsets(c, rb, R // 128).reshape(-1)].view(R // 128, 4, C)
    assert (e_col == e_col[:, :1]).all()
    assert torch.equal(e_col[:, 0].int(), fp8._e8m0(x.float().abs().view(R // 128, 128, C).amax(1)))
    # weights: one exponent per tile, identical in both directions
    w = fp8.quantize_mxfp8_ref(x, True, True, scaling="blockwise", is_weight=True)
    e_tile = fp8._e8m0(x.float().abs().view(R // 128, 128, C // 128, 128).amax((1, 3)))
    e_row_w = w.sf_row[fp8.sf_offsets(r, kb, C // 128).reshape(-1)].view(R // 128, 128, C // 128, 4)
    assert (e_row_w.int() == e_tile[:, None, :, None]).all()
    assert torch.equal(fp8.dequantize_mxfp8_ref(w.q_row, w.sf_row, False), fp8.dequantize_mxfp8_ref(w.q_col, w.sf_col, True))


def test_delayed_scaling_history_and_fallback():
    """fp8_recipe delayed: the first quantisation of a role falls back to the current maximum; after a roll the scale
    comes from the history (most recent or maximum over ``history_len`` steps, times 2^margin); values beyond the
    predicted range saturate; a slot that was not used keeps its history."""
    from primus_b200.ops import gemm

    torch.manual_seed(0)
    x = torch.randn(128, 256).bfloat16()
    try:
        gemm.set_fp8_recipe("delayed", amax_history_len=3, amax_compute_algo="max", margin=1)
        st = fp8.DELAYED
        q0 = fp8.quantize_mxfp8(x, True, False, slot_key=("w0", "x"))
        assert torch.equal(q0.sf_row, fp8.quantize_mxfp8_ref(x, True, False, scaling="tensorwise").sf_row)
        slot = st.slots[("w0", "x")]
        assert st.amax_now[slot].item() == x.float().abs().max().item()
        fp8.quantize_mxfp8(x * 0.25, True, False, slot_key=("w0", "x"))           # a second micro-batch: max is kept
        assert st.amax_now[slot].item() == x.float().abs().max().item()
        gemm.roll_fp8_scales()
        amax1 = x.float().abs().max().item()
        assert st.scale_amax[slot].item() == 2 * amax1 and st.amax_now[slot].item() == 0
        # step 2: an 8x larger tensor is scaled by the *old* maximum (x 2 margin) and saturates
        big = (x.float() * 8).bfloat16()
        q1 = fp8.quantize_mxfp8(big, True, False, slot_key=("w0", "x"))
        e_used = int(q1.sf_row[0])
        assert e_used == fp8._e8m0(torch.tensor([2 * amax1])).item()
        assert (q1.q_row.view(torch.float8_e4m3fn).float().abs() == 448).any()
        gemm.roll_fp8_scales()
        assert st.scale_amax[slot].item() == 2 * big.float().abs().max().item()      # "max" over the history
        # step 3: not used -> history stays; step 4: small tensor, the maximum of the history still rules
        gemm.roll_fp8_scales()
        assert st.history[0, slot].item() == big.float().abs().max().item()
        fp8.quantize_mxfp8((x.float() * 0.01).bfloat16(), True, False, slot_key=("w0", "x"))
        gemm.roll_fp8_scales()
        assert st.scale_amax[slot].item() == 2 * big.float().abs().max().item()
        # a tensor without a role is scaled by its current maximum
        q = fp8.quantize_mxfp8(x, True, False)
        assert torch.equal(q.sf_row, q0.sf_row)
        # most_recent picks the last rolled value
        gemm.set_fp8_recipe("delayed", amax_history_len=4, amax_compute_algo="most_recent")
        for s in (1.0, 4.0, 0.5):
            fp8.quantize_mxfp8((x.float() * s).bfloat16(), True, False, slot_key="k")
            gemm.roll_fp8_scales()
        assert fp8.DELAYED.scale_amax[fp8.DELAYED.slots["k"]].item() == (x.float() * 0.5).bfloat16().float().abs().max().item()
    finally:
        gemm.set_fp8_recipe(None)
    assert fp8.DELAYED is None and fp8.SCALING == "mxfp8"


def test_mxfp4_numerics_in_fp8_storage():
    """fp4 recipe: values lie on the E2M1 grid scaled by the block's power of two, the block maximum maps to at most
    6, ties round to even, and the stored bytes are E4M3 encodings of exactly those values."""
    torch.manual_seed(0)
    x = (torch.randn(128, 256) * torch.exp(torch.randn(128, 1))).bfloat16()
    q = fp8.quantize_mxfp8_ref(x, True, True, scaling="mxfp4")
    d = fp8.dequantize_mxfp8_ref(q.q_row, q.sf_row, False)
    e = fp8._e8m0_fp4(x.float().abs().view(128, 8, 32).amax(-1))
    scale = torch.exp2(e.float() - 127).repeat_interleave(32, 1)
    grid = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6])
    on_grid = ((d / scale).abs()[..., None] == grid).any(-1)
    assert on_grid.all()
    amax_scaled = (x.float().abs().view(128, 8, 32).amax(-1) / torch.exp2(e.float() - 127))
    assert (amax_scaled <= 6).all() and (amax_scaled[amax_scaled > 0] > 3).all()
    # error bound: half of the widest grid step (4 -> 6) in units of the block scale
    assert ((d - x.float()).abs() <= 1.0 * scale + 1e-12).all()
    v = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -2.5, 0.26, 0.74])
    assert fp8.round_to_e2m1(v).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, -2.0, 0.5, 0.5]
    from primus_b200.ops import gemm
    try:
        gemm.set_fp8_recipe("mxfp4")
        assert fp8.SCALING == "mxfp4" and torch.equal(fp8.quantize_mxfp8(x, True, False).q_row, q.q_row)
    finally:
        gemm.set_fp8_recipe(None)
