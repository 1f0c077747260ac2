"""bf16 GEMM on the tcgen05 kernel (``csrc/gemm_bf16.cu``) and the autograd linear built on it.

``gemm(a, b, a_mn, b_mn, out=..., accumulate=...)`` computes ``D = A . B^T`` where the logical
operands are A[M,K] and B[N,K]; ``a_mn`` / ``b_mn`` say that the *stored* matrix is the transpose
([K,M] / [K,N]), which the kernel consumes directly through MN-major shared-memory descriptors.

CPU tensors take a plain PyTorch fp32 path (used by the CPU test-suite and the gloo plumbing
tests); CUDA tensors always run the native kernel.

Parity: ``pt.ops.gemm`` call sites in primus/backends/megatron/core/extensions/primus_turbo.py:1182-1189
and the fused main-grad accumulation of primus/backends/megatron/core/tensor_parallel/layers.py:171-181.
"""
from __future__ import annotations

import torch

from . import _lib, autotune

_BLOCK_N_OVERRIDE: int | None = None

# ----------------------------------------------------------------------------------------------
# FP8 recipe: with ``set_fp8_recipe("mxfp8")`` every eligible GEMM (all dimensions multiples of 128, no operand
# marked ``_fp8_exempt``) quantises its operands to MXFP8 on the fly and runs on the block-scaled kernel.
# Weights are quantised (both directions) once per optimizer step; activations / gradients go through a
# two-entry cache so that a gradient used by the data- and the weight-gradient GEMM is read once.
_FP8_RECIPE: str | None = None
_WEIGHT_GEN = 0
_W_CACHE: dict = {}
_ACT_CACHE: list = []   # [(key, pinned source tensor, MXFP8Tensor)]
_PINNED: dict = {}      # key -> (placeholder tensor, MXFP8Tensor, direction whose use releases the entry)
_PINNED_MAX = 16


FP8_RECIPES = ("mxfp8", "tensorwise", "delayed", "blockwise")
FP4_RECIPES = ("mxfp4",)     # 4-bit numerics carried in FP8 storage (ops/fp8.py)


def set_fp8_recipe(recipe: str | None, amax_history_len: int = 1, amax_compute_algo: str = "most_recent",
                   margin: int = 0) -> None:
    """Select the FP8 recipe of all eligible GEMMs (None: bf16).  Every recipe stores its operands in the MXFP8 layout
    (see ``ops.fp8.SCALING``), so the GEMM kernels are the same; the three keyword arguments configure "delayed"."""
    global _FP8_RECIPE, _WEIGHT_GEN
    assert recipe in (None, "") + FP8_RECIPES + FP4_RECIPES, f"unsupported low-precision recipe {recipe!r}"
    _FP8_RECIPE = recipe or None
    from . import fp8

    fp8.SCALING = recipe or "mxfp8"
    fp8.TENSORWISE = recipe == "tensorwise"
    fp8.DELAYED = fp8.DelayedScaling(amax_history_len, amax_compute_algo, margin) if recipe == "delayed" else None
    _WEIGHT_GEN += 1        # quantised weights cached elsewhere (expert weights) are keyed on this counter
    _W_CACHE.clear()
    _ACT_CACHE.clear()
    _PINNED.clear()


def weight_generation() -> int:
    """Counter that changes whenever the optimizer (or a checkpoint load) rewrites parameters."""
    return _WEIGHT_GEN


def fp8_recipe() -> str | None:
    return _FP8_RECIPE


def bump_weight_generation() -> None:
    """Call after parameters changed in place (optimizer step, checkpoint load): cached quantised weights expire."""
    global _WEIGHT_GEN
    _WEIGHT_GEN += 1
    _ACT_CACHE.clear()


def roll_fp8_scales(group=None) -> None:
    """Once per optimizer step under the "delayed" recipe: record the step's maxima and derive the next scales."""
    from . import fp8

    if fp8.DELAYED is not None:
        fp8.DELAYED.roll(group)


def _quantized(t: torch.Tensor, direction: str, single_use: bool = False, role=None):
    """(values, scales) of ``t`` quantised along ``direction`` ("row": blocks along the last dim, "col": along dim 0).
    ``role``: (weight id, "x" | "dy") of an activation / gradient operand, the key of its delayed-scaling history."""
    from . import fp8

    if isinstance(t, torch.nn.Parameter) or getattr(t, "_is_weight", False):
        hit = _W_CACHE.get(id(t))
        if hit is None or hit[0] != _WEIGHT_GEN or hit[1] != t.data_ptr():
            hit = (_WEIGHT_GEN, t.data_ptr(),
                   fp8.quantize_mxfp8(t.detach(), True, True, is_weight=True, slot_key=(id(t), "w")))
            _W_CACHE[id(t)] = hit
        q = hit[2]
    else:
        key = (t.data_ptr(), tuple(t.shape), t._version)
        q = None
        pin = _PINNED.get(key)
        if pin is not None and getattr(pin[1], "q_" + direction) is not None:
            q = pin[1]
            if direction == pin[2]:
                del _PINNED[key]            # its last consumer
            return (q.q_row, q.sf_row) if direction == "row" else (q.q_col, q.sf_col)
        for k_, _, q_ in _ACT_CACHE:
            if k_ == key and getattr(q_, "q_" + direction) is not None:
                q = q_
                break
        if q is None:
            both = not torch.is_grad_enabled() and not single_use   # backward pass: a gradient feeds two GEMMs
            q = fp8.quantize_mxfp8(t, both or direction == "row", both or direction == "col", slot_key=role)
            _ACT_CACHE.insert(0, (key, t, q))
            del _ACT_CACHE[4:]
    return (q.q_row, q.sf_row) if direction == "row" else (q.q_col, q.sf_col)


def register_quantized(t: torch.Tensor, q, pinned: bool = False) -> None:
    """Attach an already quantised copy (both directions) to ``t``: the next GEMMs that take ``t`` as an operand use
    it instead of quantising.  ``t``'s own bf16 contents are then never read by an fp8-eligible GEMM, which lets a
    producer that can emit MXFP8 directly (fused SwiGLU backward) skip writing them.

    ``pinned``: ``t`` is a placeholder without contents (a gathered tensor that only exists in quantised form): the
    copy is kept until the GEMM that reads its last direction has run (column direction if present, else row) instead
    of living in the small recent-use cache that other quantisations push it out of.  The table is small and bounded
    (the oldest entries go first if a consumer never comes, e.g. frozen weights), so producers must not use
    placeholders while weight-gradient GEMMs are being deferred (``WGRAD_STORE.current``)."""
    key = (t.data_ptr(), tuple(t.shape), t._version)
    if pinned:
        _PINNED[key] = (t, q, "col" if q.q_col is not None else "row")
        while len(_PINNED) > _PINNED_MAX:
            del _PINNED[next(iter(_PINNED))]
        return
    _ACT_CACHE.insert(0, (key, t, q))
    del _ACT_CACHE[4:]


# set to False by code that reads gradients of linear layers outside the GEMMs (adapters), see ops/layers.py
FUSE_SWIGLU_QUANT = True


def _fp8_eligible(a, b, out, M, N, K) -> bool:
    if _FP8_RECIPE is None or (M % 128) or (N % 128) or (K % 128):
        return False
    if getattr(a, "_fp8_exempt", False) or getattr(b, "_fp8_exempt", False):
        return False
    return a.is_contiguous() and b.is_contiguous() and out.is_contiguous()


def _pick_block_n(M: int, N: int) -> int:
    if _BLOCK_N_OVERRIDE:
        return _BLOCK_N_OVERRIDE
    # measured on B200: the 128x256 tile is 35-100% faster than 128x128 on every training shape
    return 128 if N <= 128 else 256


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    max_ctas: int = 0,
    fp8: bool | None = None,
    fp8_key=None,
) -> torch.Tensor:
    """D[M,N] (+)= A . B^T with fp32 accumulation. See module docstring for layouts.  ``fp8_key``: identity of the
    weight this GEMM belongs to when it is not operand B (weight-gradient GEMMs), for delayed scaling."""
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"K mismatch: {K} vs {Kb}"
    if out_dtype is None:
        out_dtype = torch.bfloat16 if a.is_cuda else a.dtype
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N)
        out_dtype = out.dtype
    if accumulate:
        assert out_dtype == torch.float32, "accumulate mode writes fp32"

    if not a.is_cuda:
        A = a.float().t() if a_mn else a.float()
        B = b.float() if b_mn else b.float().t()
        r = A @ B
        if accumulate:
            out.add_(r)
        else:
            out.copy_(r.to(out_dtype))
        return out

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    mode = 0 if out_dtype == torch.bfloat16 else (2 if accumulate else 1)
    use_fp8 = fp8 is not False and _fp8_eligible(a, b, out, M, N, K)
    tuned = None
    if autotune.active() and not _BLOCK_N_OVERRIDE:
        tuned = autotune.lookup(autotune.make_key("mxfp8" if use_fp8 else "bf16", M, N, K, a_mn, b_mn, mode))
    if use_fp8:
        # operand roles (delayed scaling keeps one history per weight and role): fprop x . W, dgrad dy . W, wgrad dy . x
        wid = fp8_key if fp8_key is not None else id(b)
        aq, asf = _quantized(a, "col" if a_mn else "row", role=(wid, "x" if not (a_mn or b_mn) else "dy"))
        bq, bsf = _quantized(b, "col" if b_mn else "row", single_use=a_mn and b_mn,   # wgrad: B is the saved input
                             role=(wid, "x"))
        from . import fp8 as _fp8

        _fp8.launch_gemm(aq, asf, bq, bsf, out, M, N, K, a_mn, b_mn, mode, tuned.get("block_n") if tuned else None,
                         max_ctas or (tuned.get("max_ctas", 0) if tuned else 0),
                         tuned.get("two_cta") if tuned else None)
        return out
    launch_bf16(a, b, out, M, N, K, a_mn, b_mn, mode, (tuned.get("block_n") if tuned else None) or _pick_block_n(M, N),
                max_ctas or (tuned.get("max_ctas", 0) if tuned else 0))
    return out


def launch_bf16(a, b, out, M: int, N: int, K: int, a_mn: bool, b_mn: bool, mode: int, block_n: int,
                max_ctas: int = 0) -> None:
    """Raw launch of the bf16 tcgen05 GEMM with explicit tile options (the autotuner times candidates through it)."""
    _lib.call(
        "gemm_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), mode, block_n, max_ctas, _lib.status_word(a.device),
    )


class LinearFn(torch.autograd.Function):
    """y = x W^T.  Backward: dx = dy W (MN-major B), dW accumulated in fp32 into ``main_grad``
    when the weight owns one (Megatron ``main_grad`` convention), else returned as a bf16 grad."""

    @staticmethod
    def forward(ctx, x, weight):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y = gemm(x2, weight)
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = shape
        ctx.weight_ref = weight
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = wgrad(dy2, x2, ctx.weight_ref)
        return dx, dw


class WGradStore:
    """Deferred weight-gradient GEMMs for zero-bubble pipeline schedules: while a ``B`` node runs
    (``begin(key)`` .. ``end()``), linear layers queue their dW GEMM instead of executing it; the matching
    ``W`` node replays the queue with ``flush(key)``.  (Role of the reference's ``WGradRunningCache``,
    primus/core/pipeline_parallel/handler/wgrad_handler.py:17-78.)"""

    def __init__(self):
        self.current = None
        self.queues: dict = {}

    def begin(self, key):
        self.current = key
        self.queues.setdefault(key, [])

    def end(self):
        self.current = None

    def put(self, dy2, x2, weight) -> bool:
        if self.current is None or getattr(weight, "main_grad", None) is None:
            return False
        self.queues[self.current].append((dy2, x2, weight))
        return True

    def flush(self, key):
        with torch.no_grad():
            for dy2, x2, weight in self.queues.pop(key, []):
                _wgrad_into_main_grad(dy2.detach(), x2.detach(), weight)

    def flush_all(self):
        for k in list(self.queues):
            self.flush(k)


WGRAD_STORE = WGradStore()


def _wgrad_into_main_grad(dy2, x2, weight):
    gemm(dy2, x2, a_mn=True, b_mn=True, out=weight.main_grad, accumulate=True,
         fp8=False if getattr(weight, "_fp8_exempt", False) else None, fp8_key=id(weight))
    weight.grad_added_to_main_grad = True
    cb = getattr(weight, "_grad_ready_cb", None)
    if cb is not None:
        cb(weight)


def wgrad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor):
    """dW = dy^T x. Accumulates into ``weight.main_grad`` (fp32) if present and returns None;
    otherwise returns the gradient in the weight's dtype."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        if not WGRAD_STORE.put(dy2, x2, weight):
            _wgrad_into_main_grad(dy2, x2, weight)
        return None
    if dy2.is_cuda:
        return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype,
                    fp8=False if getattr(weight, "_fp8_exempt", False) else None, fp8_key=id(weight))
    return (dy2.float().t() @ x2.float()).to(weight.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return LinearFn.apply(x, weight)


autotune.configure_from_env()
