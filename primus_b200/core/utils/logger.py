"""Per-rank logging: stderr sink (rank-aware) plus ``<exp_root>/logs/<module>/rank-<r>/{debug,info,
warning,error}.log`` files; ``PRIMUS_LOG_LEVEL`` overrides the configured stderr level
(primus/core/utils/logger.py:62-251, primus/core/runtime/logging.py:57-158 in the reference, which uses
loguru; this implementation is on the standard ``logging`` module)."""
from __future__ import annotations

import logging
import os
import sys
from typing import Optional

_LOGGER: Optional[logging.Logger] = None
_RANK = 0
_WORLD = 1


class _RankFilter(logging.Filter):
    def filter(self, record):
        record.rank = _RANK
        record.world = _WORLD
        return True


def setup_logger(exp_root: Optional[str] = None, module: str = "pre_trainer", rank: int = 0, world: int = 1,
                 stderr_level: str = "INFO", file_level: str = "DEBUG") -> logging.Logger:
    global _LOGGER, _RANK, _WORLD
    _RANK, _WORLD = rank, world
    stderr_level = os.environ.get("PRIMUS_LOG_LEVEL", stderr_level).upper()
    lg = logging.getLogger("primus_b200")
    lg.setLevel(logging.DEBUG)
    lg.handlers.clear()
    lg.propagate = False
    fmt = logging.Formatter("[%(asctime)s][rank-%(rank)d/%(world)d][%(levelname)s] %(message)s", "%Y%m%d %H:%M:%S")
    h = logging.StreamHandler(sys.stderr)
    h.setLevel(getattr(logging, stderr_level, logging.INFO))
    h.setFormatter(fmt)
    h.addFilter(_RankFilter())
    lg.addHandler(h)
    if exp_root:
        d = os.path.join(exp_root, "logs", module, f"rank-{rank}")
        os.makedirs(d, exist_ok=True)
        for name in ("debug", "info", "warning", "error"):
            lvl = getattr(logging, name.upper())
            if lvl < getattr(logging, file_level.upper(), logging.DEBUG):
                continue
            fh = logging.FileHandler(os.path.join(d, f"{name}.log"))
            fh.setLevel(lvl)
            fh.setFormatter(fmt)
            fh.addFilter(_RankFilter())
            lg.addHandler(fh)
    _LOGGER = lg
    return lg


def get_logger() -> logging.Logger:
    return _LOGGER or setup_logger()


def log_rank_0(msg: str, level=logging.INFO):
    if _RANK == 0:
        get_logger().log(level, msg)


def log_rank_last(msg: str, level=logging.INFO):
    if _RANK == _WORLD - 1:
        get_logger().log(level, msg)


def log_rank_all(msg: str, level=logging.INFO):
    get_logger().log(level, msg)


def log_dict_aligned(title: str, d: dict, log=log_rank_0):
    """One ``key ....... value`` line per entry, keys sorted and dot-padded to a common width."""
    if not d:
        return
    w = max(len(str(k)) for k in d) + 2
    log(f"-------- {title} --------")
    for k in sorted(d):
        log(f"  {str(k).ljust(w, '.')} {d[k]}")
