"""Tile-configuration cache for the tcgen05 GEMM kernels.

The GEMM launchers take a small set of launch options (N-tile 128 / 256, one-CTA or CTA-pair kernel, a CTA cap) and the
best choice depends on the problem shape.  This module keeps a table ``key -> options`` where
``key = (kind, M, N, K, a_mn, b_mn, mode)`` (kind: ``bf16`` / ``mxfp8``; mode: bf16 out / fp32 out / fp32 accumulate) and
offers the three-stage workflow of the reference's GEMM tuning plus an online mode:

1. **dump** (``PRIMUS_B200_GEMM_TUNING_STAGE=1`` or ``record_shapes(True)``): a short job records every GEMM key it
   launches; ``dump_shapes(path)`` (called at exit) writes them as JSON, one file per rank.
2. **tune offline** (``python -m primus_b200.tools.tune_gemm --shapes ... --out tuned.json``): every candidate of
   every recorded key is timed with CUDA events over rotating operands larger than L2; the fastest wins.
3. **use** (``PRIMUS_B200_GEMM_TUNING_FILE=tuned.json`` or ``load(path)``): ``ops.gemm`` asks ``lookup(key)`` before
   each launch and falls back to its built-in heuristic for unknown keys.

Online mode (``use_turbo_autotune`` -> ``PRIMUS_B200_AUTOTUNE=1``): the first time a key is launched its candidates are
timed on scratch operands of the same shape and the winner is cached for the life of the process (and written to
``PRIMUS_B200_GEMM_TUNING_SAVE`` at exit when set).  Everything is off under ``PRIMUS_DETERMINISTIC=1``.

Role of the reference's hipBLASLt tuning workflow (``PRIMUS_HIPBLASLT_TUNING`` stages in
runner/helpers/hooks/train/pretrain/prepare_experiment.sh:199-266, examples/offline_tune/offline_tune_gemm.py) and of
Primus-Turbo's ``PRIMUS_TURBO_AUTO_TUNE`` switch (primus/backends/megatron/patches/args/rocm_arg_validation.py:112-114).
"""
from __future__ import annotations

import atexit
import json
import os
import socket
from typing import Callable, Iterable, Optional

Key = tuple  # (kind, M, N, K, a_mn, b_mn, mode)

_TABLE: dict[Key, dict] = {}
_SEEN: dict[Key, int] = {}
_RECORD = False
_ONLINE = False
_TIMER: Optional[Callable] = None      # test hook: (key, options) -> seconds
_DIRTY = False


def _deterministic() -> bool:
    return os.environ.get("PRIMUS_DETERMINISTIC", "0") == "1"


def make_key(kind: str, M: int, N: int, K: int, a_mn: bool, b_mn: bool, mode: int) -> Key:
    return (kind, int(M), int(N), int(K), int(bool(a_mn)), int(bool(b_mn)), int(mode))


def _key_str(key: Key) -> str:
    return ":".join(str(x) for x in key)


def _key_from_str(s: str) -> Key:
    p = s.split(":")
    return (p[0],) + tuple(int(x) for x in p[1:])


def candidates(key: Key) -> list[dict]:
    """Launch options worth timing for ``key`` (the first entry is the built-in default)."""
    kind, M, N, K = key[:4]
    out = [{"block_n": 256 if N > 128 else 128}]
    if N > 128:
        out.append({"block_n": 128})
    if kind == "mxfp8" and M % 256 == 0 and N % 256 == 0 and M >= 256 and N >= 256:
        out.append({"two_cta": True})
    return out


# ------------------------------------------------------------------------------------------------ table
def active() -> bool:
    """False when no table, recording or online tuning is in use: callers skip the key construction entirely."""
    return bool(_TABLE) or _RECORD or _ONLINE


def lookup(key: Key) -> Optional[dict]:
    """Options for ``key`` or None (use the heuristic).  Records the key in stage 1 and tunes it in online mode."""
    if _RECORD:
        _SEEN[key] = _SEEN.get(key, 0) + 1
    if _deterministic():
        return None
    hit = _TABLE.get(key)
    if hit is None and _ONLINE:
        hit = tune_key(key)
    return hit


def set_entry(key: Key, options: dict, time_s: Optional[float] = None) -> None:
    global _DIRTY
    _TABLE[key] = dict(options, **({"time_us": round(time_s * 1e6, 3)} if time_s is not None else {}))
    _DIRTY = True


def clear() -> None:
    global _DIRTY
    _TABLE.clear()
    _SEEN.clear()
    _DIRTY = False


def table() -> dict:
    return dict(_TABLE)


def load(path: str) -> int:
    """Merge a tuning file into the table; returns the number of entries read."""
    with open(path) as f:
        doc = json.load(f)
    for k, v in doc.get("entries", {}).items():
        _TABLE[_key_from_str(k)] = v
    return len(doc.get("entries", {}))


def save(path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump({"version": 1, "device": _device_name(), "entries": {_key_str(k): v for k, v in sorted(_TABLE.items())}},
                  f, indent=1)


def _device_name() -> str:
    try:
        import torch

        return torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    except Exception:
        return "unknown"


# ------------------------------------------------------------------------------------------------ stage 1: shapes
def record_shapes(on: bool = True) -> None:
    global _RECORD
    _RECORD = on


def seen_shapes() -> dict:
    return dict(_SEEN)


def dump_shapes(path: Optional[str] = None) -> Optional[str]:
    """Write the recorded keys (with call counts) as JSON; default file name carries host and rank like the
    reference's per-node shape dumps."""
    if not _SEEN:
        return None
    if path is None:
        d = os.environ.get("PRIMUS_B200_GEMM_SHAPE_DIR", "gemm_shape")
        path = os.path.join(d, f"gemm_shapes_{socket.gethostname()}_rank{os.environ.get('RANK', '0')}.json")
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump({"version": 1, "shapes": {_key_str(k): n for k, n in sorted(_SEEN.items())}}, f, indent=1)
    return path


def read_shapes(paths: Iterable[str]) -> dict:
    """Union of several shape dumps (call counts summed)."""
    out: dict = {}
    for p in paths:
        with open(p) as f:
            for k, n in json.load(f).get("shapes", {}).items():
                key = _key_from_str(k)
                out[key] = out.get(key, 0) + int(n)
    return out


# ------------------------------------------------------------------------------------------------ stage 2: timing
def _time_candidate(key: Key, options: dict, iters: int = 8) -> float:
    """Median device time of one launch of ``key`` with ``options`` on scratch operands (rotated through enough copies
    to exceed L2 for small problems)."""
    if _TIMER is not None:
        return _TIMER(key, options)
    import torch

    from . import _lib, fp8
    from . import gemm as G

    kind, M, N, K, a_mn, b_mn, mode = key
    dev = torch.device("cuda", torch.cuda.current_device())
    elem = 1 if kind == "mxfp8" else 2
    per_set = (M * K + N * K) * elem + M * N * (2 if mode == 0 else 4)
    copies = max(2, min(8, (192 << 20) // max(per_set, 1) + 1))
    out_dtype = torch.bfloat16 if mode == 0 else torch.float32
    sets = []
    for _ in range(copies):
        a_shape = (K, M) if a_mn else (M, K)
        b_shape = (K, N) if b_mn else (N, K)
        if kind == "mxfp8":
            a = torch.randint(0, 120, a_shape, dtype=torch.uint8, device=dev)
            b = torch.randint(0, 120, b_shape, dtype=torch.uint8, device=dev)
            sa = torch.full((M * K // 32,), 127, dtype=torch.uint8, device=dev)
            sb = torch.full((N * K // 32,), 127, dtype=torch.uint8, device=dev)
            sets.append((a, sa, b, sb, torch.zeros(M, N, dtype=out_dtype, device=dev)))
        else:
            a = torch.randn(a_shape, device=dev, dtype=torch.bfloat16)
            b = torch.randn(b_shape, device=dev, dtype=torch.bfloat16)
            sets.append((a, b, torch.zeros(M, N, dtype=out_dtype, device=dev)))

    def launch(i):
        s = sets[i % copies]
        if kind == "mxfp8":
            fp8.launch_gemm(s[0], s[1], s[2], s[3], s[4], M, N, K, bool(a_mn), bool(b_mn), mode,
                            options.get("block_n"), options.get("max_ctas", 0), bool(options.get("two_cta", False)))
        else:
            G.launch_bf16(s[0], s[1], s[2], M, N, K, bool(a_mn), bool(b_mn), mode,
                          options.get("block_n") or G._pick_block_n(M, N), options.get("max_ctas", 0))

    for i in range(3):
        launch(i)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch(i)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e-3)
    _lib.check_status()
    times.sort()
    return times[len(times) // 2]


def tune_key(key: Key) -> dict:
    """Time every candidate of ``key``, store and return the fastest."""
    best, best_t, all_t = None, None, {}
    for opt in candidates(key):
        try:
            t = _time_candidate(key, opt)
        except Exception as e:          # a candidate the kernel rejects for this shape is simply not eligible
            all_t[json.dumps(opt, sort_keys=True)] = f"rejected: {type(e).__name__}"
            continue
        all_t[json.dumps(opt, sort_keys=True)] = round(t * 1e6, 3)
        if best_t is None or t < best_t:
            best, best_t = opt, t
    if best is None:
        best, best_t = candidates(key)[0], None
    set_entry(key, best, best_t)
    _TABLE[key]["candidates_us"] = all_t
    return _TABLE[key]


def tune_shapes(shapes: Iterable[Key], log: Optional[Callable[[str], None]] = None) -> dict:
    for key in shapes:
        r = tune_key(key)
        if log is not None:
            log(f"{_key_str(key)} -> {json.dumps({k: v for k, v in r.items() if k != 'candidates_us'})}")
    return table()


# ------------------------------------------------------------------------------------------------ environment
def configure_from_env() -> None:
    """Apply the environment policy once at import of ``ops.gemm``."""
    global _ONLINE
    if _deterministic():
        return
    stage = os.environ.get("PRIMUS_B200_GEMM_TUNING_STAGE", "")
    if stage == "1":
        record_shapes(True)
        atexit.register(dump_shapes)
    f = os.environ.get("PRIMUS_B200_GEMM_TUNING_FILE")
    if f and os.path.exists(f):
        load(f)
    if os.environ.get("PRIMUS_B200_AUTOTUNE", "0") == "1":
        _ONLINE = True
        out = os.environ.get("PRIMUS_B200_GEMM_TUNING_SAVE")
        if out:
            atexit.register(lambda: save(out) if _DIRTY else None)


def set_online(on: bool) -> None:
    global _ONLINE
    _ONLINE = on and not _deterministic()
