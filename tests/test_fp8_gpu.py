"""MXFP8 quantisation and block-scaled GEMM kernels vs plain PyTorch restatements."""
import pytest
import torch

from primus_b200.ops import _lib, fp8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("R,C", [(128, 128), (256, 384), (1024, 512)])
def test_quantize_matches_reference_bitwise(R, C):
    torch.manual_seed(0)
    x = (torch.randn(R, C, device="cuda") * torch.exp(torch.randn(R, 1, device="cuda") * 3)).bfloat16()
    x[5, 32:64] = 0
    q = fp8.quantize_mxfp8(x)
    ref = fp8.quantize_mxfp8_ref(x)
    for name in ("q_row", "sf_row", "q_col", "sf_col"):
        assert torch.equal(getattr(q, name), getattr(ref, name)), name
    for colwise, qq, sf in ((False, q.q_row, q.sf_row), (True, q.q_col, q.sf_col)):
        deq = fp8.dequantize_mxfp8(qq, sf, colwise)
        assert torch.equal(deq, fp8.dequantize_mxfp8_ref(qq, sf, colwise))
        err = (deq - x.float()).abs()
        assert (err <= x.float().abs() * 0.0626 + 1e-30).all() or err.max() <= 0.07 * x.float().abs().max()


@pytest.mark.parametrize("R,C", [(128, 128), (1024, 512), (4096, 2048)])
def test_tensorwise_quantiser_matches_reference_bitwise(R, C):
    """One power-of-two scale for the whole tensor (maximum reduction + quantiser), MXFP8 storage layout."""
    torch.manual_seed(1)
    x = (torch.randn(R, C, device="cuda") * torch.exp(torch.randn(R, 1, device="cuda") * 2)).bfloat16()
    q = fp8.quantize_mxfp8(x, True, True, tensorwise=True)
    ref = fp8.quantize_mxfp8_ref(x, True, True, tensorwise=True)
    torch.cuda.synchronize()
    _lib.check_status()
    for name in ("q_row", "sf_row", "q_col", "sf_col"):
        assert torch.equal(getattr(q, name), getattr(ref, name)), name
    assert q.sf_row.unique().numel() == 1
    only_row = fp8.quantize_mxfp8(x, True, False, tensorwise=True)
    assert only_row.q_col is None and torch.equal(only_row.q_row, ref.q_row)


@pytest.mark.parametrize("R,C", [(128, 128), (512, 384), (2048, 1024)])
@pytest.mark.parametrize("is_weight", [False, True])
def test_blockwise_quantiser_matches_reference_bitwise(R, C, is_weight):
    """One power-of-two scale per 1 x 128 vector (activations) or 128 x 128 tile (weights), MXFP8 storage layout."""
    torch.manual_seed(2)
    x = (torch.randn(R, C, device="cuda") * torch.exp(torch.randn(R, 1, device="cuda") * 2)).bfloat16()
    x[3, 0:128] = 0
    q = fp8.quantize_mxfp8(x, True, True, scaling="blockwise", is_weight=is_weight)
    ref = fp8.quantize_mxfp8_ref(x, True, True, scaling="blockwise", is_weight=is_weight)
    torch.cuda.synchronize()
    _lib.check_status()
    for name in ("q_row", "sf_row", "q_col", "sf_col"):
        assert torch.equal(getattr(q, name), getattr(ref, name)), name
    only_col = fp8.quantize_mxfp8(x, False, True, scaling="blockwise", is_weight=is_weight)
    assert only_col.q_row is None and torch.equal(only_col.q_col, ref.q_col)


@pytest.mark.parametrize("R,C", [(128, 128), (1024, 512)])
def test_mxfp4_quantiser_matches_reference_bitwise(R, C):
    """E2M1 values with a power-of-two scale per 32 elements, stored as E4M3 bytes."""
    torch.manual_seed(5)
    x = (torch.randn(R, C, device="cuda") * torch.exp(torch.randn(R, 1, device="cuda") * 2)).bfloat16()
    x[0, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], device="cuda").bfloat16()   # ties, max = 6
    x[0, 8:32] = 0
    q = fp8.quantize_mxfp8(x, True, True, scaling="mxfp4")
    ref = fp8.quantize_mxfp8_ref(x, True, True, scaling="mxfp4")
    torch.cuda.synchronize()
    _lib.check_status()
    for name in ("q_row", "sf_row", "q_col", "sf_col"):
        assert torch.equal(getattr(q, name), getattr(ref, name)), name


def test_delayed_quantiser_uses_history_and_records_the_maximum():
    from primus_b200.ops import gemm

    torch.manual_seed(3)
    x = torch.randn(512, 256, device="cuda").bfloat16()
    try:
        gemm.set_fp8_recipe("delayed", amax_history_len=2, amax_compute_algo="max")
        st = fp8.DELAYED
        q0 = fp8.quantize_mxfp8(x, True, True, slot_key="a")                 # empty history: current maximum
        ref0 = fp8.quantize_mxfp8_ref(x, True, True, scaling="tensorwise")
        assert torch.equal(q0.q_row, ref0.q_row) and torch.equal(q0.sf_col, ref0.sf_col)
        slot = st.slots["a"]
        assert st.amax_now[slot].item() == x.float().abs().max().item()
        gemm.roll_fp8_scales()
        big = (x.float() * 16).bfloat16()
        q1 = fp8.quantize_mxfp8(big, True, True, slot_key="a")               # scaled by the previous step's maximum
        ref1 = fp8.quantize_mxfp8_ref(big, True, True, scaling="delayed", scale_amax=st.scale_amax[slot])
        for name in ("q_row", "sf_row", "q_col", "sf_col"):
            assert torch.equal(getattr(q1, name), getattr(ref1, name)), name
        assert (q1.q_row.view(torch.float8_e4m3fn).float().abs() == 448).any()
        assert st.amax_now[slot].item() == big.float().abs().max().item()
        torch.cuda.synchronize()
        _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)


def _ref_gemm(aq, asf, a_col, bq, bsf, b_col, a_mn, b_mn):
    A = fp8.dequantize_mxfp8(aq, asf, a_col)
    B = fp8.dequantize_mxfp8(bq, bsf, b_col)
    A = A.t() if a_mn else A
    B = B.t() if b_mn else B
    return A @ B.t()


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 128, 256), (256, 512, 512, 256), (384, 128, 256, 128),
                                      (512, 768, 1024, 256), (256, 384, 384, 128)])
def test_gemm_fprop_layout(M, N, K, bn):
    torch.manual_seed(1)
    a = (torch.randn(M, K, device="cuda") * 2).bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    aq, bq = fp8.quantize_mxfp8(a, True, False), fp8.quantize_mxfp8(b, True, False)
    out = fp8.gemm_mxfp8(aq.q_row, aq.sf_row, bq.q_row, bq.sf_row, M, N, K, block_n=bn)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref_gemm(aq.q_row, aq.sf_row, False, bq.q_row, bq.sf_row, False, False, False)
    err = (out.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item(), (err, ref.abs().max().item())


@pytest.mark.parametrize("T,N,K", [(256, 256, 384), (512, 384, 256)])
def test_linear_fwd_bwd_against_dequantised_reference(T, N, K):
    torch.manual_seed(2)
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    dy = torch.randn(T, N, device="cuda").bfloat16()
    y = fp8.linear_mxfp8(x, w)
    y.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xq, wq, dyq = fp8.quantize_mxfp8(x.detach()), fp8.quantize_mxfp8(w.detach()), fp8.quantize_mxfp8(dy)
    y_ref = _ref_gemm(xq.q_row, xq.sf_row, False, wq.q_row, wq.sf_row, False, False, False)
    dx_ref = fp8.dequantize_mxfp8(dyq.q_row, dyq.sf_row, False) @ fp8.dequantize_mxfp8(wq.q_col, wq.sf_col, True)
    dw_ref = fp8.dequantize_mxfp8(dyq.q_col, dyq.sf_col, True).t() @ fp8.dequantize_mxfp8(xq.q_col, xq.sf_col, True)
    for got, ref, name in ((y, y_ref, "y"), (x.grad, dx_ref, "dx"), (w.grad, dw_ref, "dw")):
        err = (got.float() - ref).abs().max().item()
        assert err <= 1.5e-2 * ref.abs().max().item(), (name, err, ref.abs().max().item())
    # and close to the bf16 result (quantisation noise only)
    y_bf = x.detach().float() @ w.detach().float().t()
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), y_bf.flatten(), dim=0).item()
    assert cos > 0.995, cos


def test_wgrad_accumulates_into_main_grad():
    T, N, K = 256, 256, 256
    torch.manual_seed(3)
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    w.main_grad = torch.ones(N, K, dtype=torch.float32, device="cuda")
    dy = torch.randn(T, N, device="cuda").bfloat16()
    fp8.linear_mxfp8(x, w).backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xq, dyq = fp8.quantize_mxfp8(x), fp8.quantize_mxfp8(dy)
    dw_ref = fp8.dequantize_mxfp8(dyq.q_col, dyq.sf_col, True).t() @ fp8.dequantize_mxfp8(xq.q_col, xq.sf_col, True)
    err = (w.main_grad - 1.0 - dw_ref).abs().max().item()
    assert err <= 1e-2 * dw_ref.abs().max().item(), err
    assert w.grad is None


def test_model_training_with_mxfp8_recipe_tracks_bf16():
    """Same tiny model, same data: the MXFP8 recipe's loss trajectory stays close to the bf16 one."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    losses = {}
    try:
        for recipe, kind in ((None, "mxfp8"), ("e4m3", "mxfp8"), ("e4m3", "tensorwise"), ("e4m3", "blockwise"),
                             ("e4m3", "delayed")):
            mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2,
                                   num_query_groups=2, vocab_size=1024, params_dtype="bf16", seq_length=256, fp8=recipe,
                                   fp8_recipe=kind)
            tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=6, lr=2e-3,
                             lr_decay_style="constant", weight_decay=0.0, clip_grad=1.0, log_interval=1)
            torch.manual_seed(0)
            tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
            assert gemm.fp8_recipe() == (kind if recipe else None)
            losses[(recipe, kind)] = tr.train()
            torch.cuda.synchronize()
            _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)
    a, b, c = losses[(None, "mxfp8")], losses[("e4m3", "mxfp8")], losses[("e4m3", "tensorwise")]
    assert all(abs(x - y) <= 0.02 * abs(x) for x, y in zip(a, b)), (a, b)
    assert all(abs(x - y) <= 0.03 * abs(x) for x, y in zip(a, c)), (a, c)
    for kind in ("blockwise", "delayed"):
        d = losses[("e4m3", kind)]
        assert all(abs(x - y) <= 0.03 * abs(x) for x, y in zip(a, d)), (kind, a, d)


def test_model_training_with_mxfp4_numerics_tracks_bf16():
    """MXFP4 numerics on every linear-layer GEMM (no stochastic rounding, no Hadamard transform): the loss stays
    within 3 % of the bf16 trajectory on the tiny model (random mock data: neither run's loss falls much)."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    out = {}
    try:
        for fp4 in (None, "e2m1"):
            mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2,
                                   num_query_groups=2, vocab_size=1024, params_dtype="bf16", seq_length=256, fp4=fp4)
            tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=8, lr=2e-3,
                             lr_decay_style="constant", weight_decay=0.0, clip_grad=1.0, log_interval=1)
            torch.manual_seed(0)
            tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
            assert gemm.fp8_recipe() == ("mxfp4" if fp4 else None)
            out[fp4] = tr.train()
            torch.cuda.synchronize()
            _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)
    a, b = out[None], out["e2m1"]
    assert a != b and all(abs(x - y) <= 0.03 * abs(x) for x, y in zip(a, b)), (a, b)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 512, 512), (384, 768, 256), (1024, 1280, 1024), (384, 384, 256),
                                   (640, 896, 384), (2048, 1536, 2176)])
def test_cta_pair_gemm_all_layouts(M, N, K):
    """256 x 256 tiles on CTA pairs: forward, data-gradient and weight-gradient operand layouts."""
    torch.manual_seed(4)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    dy = torch.randn(M, N, device="cuda").bfloat16()
    xq, wq, dyq = fp8.quantize_mxfp8(x), fp8.quantize_mxfp8(w), fp8.quantize_mxfp8(dy)
    y = fp8.gemm_mxfp8(xq.q_row, xq.sf_row, wq.q_row, wq.sf_row, M, N, K, two_cta=True)
    dx = fp8.gemm_mxfp8(dyq.q_row, dyq.sf_row, wq.q_col, wq.sf_col, M, K, N, b_mn=True, two_cta=True)
    dw = torch.ones(N, K, dtype=torch.float32, device="cuda")
    fp8.gemm_mxfp8(dyq.q_col, dyq.sf_col, xq.q_col, xq.sf_col, N, K, M, a_mn=True, b_mn=True, out=dw, accumulate=True,
                   two_cta=True)
    torch.cuda.synchronize()
    _lib.check_status()
    y_ref = _ref_gemm(xq.q_row, xq.sf_row, False, wq.q_row, wq.sf_row, False, False, False)
    dx_ref = fp8.dequantize_mxfp8(dyq.q_row, dyq.sf_row, False) @ fp8.dequantize_mxfp8(wq.q_col, wq.sf_col, True)
    dw_ref = fp8.dequantize_mxfp8(dyq.q_col, dyq.sf_col, True).t() @ fp8.dequantize_mxfp8(xq.q_col, xq.sf_col, True)
    for got, ref, name in ((y, y_ref, "y"), (dx, dx_ref, "dx"), (dw - 1.0, dw_ref, "dw")):
        err = (got.float() - ref).abs().max().item()
        assert err <= 1.5e-2 * ref.abs().max().item(), (name, err, ref.abs().max().item())


def test_fused_swiglu_quantisation_is_bitwise_equal_to_unfused():
    """SwiGLU kernels that emit MXFP8 directly (forward activation, backward input gradient) must reproduce the
    un-fused bf16 -> quantise path exactly: same loss trajectory bit for bit."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    out = {}
    try:
        for fuse in (True, False):
            gemm.FUSE_SWIGLU_QUANT = fuse
            mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2,
                                   num_query_groups=2, vocab_size=1024, params_dtype="bf16", seq_length=256, fp8="e4m3",
                                   fp8_recipe="mxfp8")
            tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=4, lr=2e-3,
                             lr_decay_style="constant", weight_decay=0.0, clip_grad=1.0, log_interval=1)
            torch.manual_seed(0)
            tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
            out[fuse] = tr.train()
            torch.cuda.synchronize()
            _lib.check_status()
    finally:
        gemm.FUSE_SWIGLU_QUANT = True
        gemm.set_fp8_recipe(None)
    assert out[True] == out[False], out


@pytest.mark.parametrize("counts,N,K", [([100, 0, 300, 129, 1, 128], 384, 256), ([512, 512], 512, 1024),
                                        ([0, 0, 7], 128, 128), ([700, 33, 260, 5], 1408, 2048)])
def test_grouped_gemm_mxfp8_against_dequantised_reference(counts, N, K):
    """Per-expert MXFP8 GEMMs (forward, data gradient, weight gradient) vs fp32 matmuls of the dequantised operands."""
    from primus_b200.ops import gemm
    from primus_b200.ops import moe as M

    E, R = len(counts), sum(counts)
    s = M.build_schedule(torch.tensor(counts, dtype=torch.int32, device="cuda"), M.rows_capacity(R, E))
    rs, pd = s.row_start.tolist(), s.padded.tolist()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.zeros(s.rows_cap, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.zeros(s.rows_cap, N, device="cuda", dtype=torch.bfloat16)
    for e, c in enumerate(counts):
        x[rs[e]:rs[e] + c] = torch.randn(c, K, device="cuda", generator=g).bfloat16()
        dy[rs[e]:rs[e] + c] = torch.randn(c, N, device="cuda", generator=g).bfloat16()
    w = torch.nn.Parameter((torch.randn(E, N, K, device="cuda", generator=g) * 0.05).bfloat16())
    w.main_grad = torch.ones(E, N, K, device="cuda")
    gemm.set_fp8_recipe("mxfp8")
    try:
        xg = x.clone().requires_grad_()
        y = M.grouped_linear(xg, w, s)
        y.backward(dy)
        torch.cuda.synchronize()
        _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)
    xq, dyq = fp8.quantize_mxfp8(x), fp8.quantize_mxfp8(dy)
    wq = fp8.quantize_mxfp8(w.detach().view(E * N, K))
    x_r, x_c = fp8.dequantize_mxfp8(xq.q_row, xq.sf_row, False), fp8.dequantize_mxfp8(xq.q_col, xq.sf_col, True)
    dy_r, dy_c = fp8.dequantize_mxfp8(dyq.q_row, dyq.sf_row, False), fp8.dequantize_mxfp8(dyq.q_col, dyq.sf_col, True)
    w_r = fp8.dequantize_mxfp8(wq.q_row, wq.sf_row, False).view(E, N, K)
    w_c = fp8.dequantize_mxfp8(wq.q_col, wq.sf_col, True).view(E, N, K)
    for e in range(E):
        sl = slice(rs[e], rs[e] + pd[e])
        if pd[e]:
            y_ref = x_r[sl].float() @ w_r[e].float().t()
            dx_ref = dy_r[sl].float() @ w_c[e].float()
            torch.testing.assert_close(y[sl].float(), y_ref, rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(xg.grad[sl].float(), dx_ref, rtol=2e-2, atol=2e-2)
        dw_ref = 1.0 + dy_c[sl].float().t() @ x_c[sl].float()
        torch.testing.assert_close(w.main_grad[e], dw_ref, rtol=1e-3, atol=1e-2)


def test_moe_model_with_mxfp8_recipe_tracks_bf16():
    """MoE model (grouped expert GEMMs in MXFP8 under the recipe): loss trajectory stays close to bf16."""
    from primus_b200.engine.trainer import TrainConfig, Trainer
    from primus_b200.models.config import TransformerConfig
    from primus_b200.ops import gemm
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    losses = {}
    try:
        for recipe in (None, "e4m3"):
            mc = TransformerConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=2,
                                   num_query_groups=2, vocab_size=1024, params_dtype="bf16", seq_length=512,
                                   num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=256, moe_layer_freq=[0, 1],
                                   moe_aux_loss_coeff=1e-2, fp8=recipe, fp8_recipe="mxfp8")
            tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=512, train_iters=6, lr=2e-3,
                             lr_decay_style="constant", weight_decay=0.0, clip_grad=1.0, log_interval=1)
            torch.manual_seed(0)
            tr = Trainer(mc, tc, device="cuda", log_fn=lambda s: None)
            losses[recipe] = tr.train()
            torch.cuda.synchronize()
            _lib.check_status()
    finally:
        gemm.set_fp8_recipe(None)
    a, b = losses[None], losses["e4m3"]
    assert all(abs(x - y) <= 0.03 * abs(x) for x, y in zip(a, b)), (a, b)
