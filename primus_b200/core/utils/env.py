"""torchrun environment helpers (primus/core/utils/env.py:41-56 in the reference)."""
from __future__ import annotations

import os


def get_torchrun_env() -> dict:
    e = os.environ
    return {"rank": int(e.get("RANK", 0)), "world_size": int(e.get("WORLD_SIZE", 1)),
            "local_rank": int(e.get("LOCAL_RANK", 0)), "local_world_size": int(e.get("LOCAL_WORLD_SIZE", 1)),
            "master_addr": e.get("MASTER_ADDR", "127.0.0.1"), "master_port": int(e.get("MASTER_PORT", 29500))}


def setup_training_env(exp_root: str | None = None) -> None:
    """Cache locations for tokenizers / datasets default under the data path."""
    base = os.environ.get("DATA_PATH") or (os.path.join(exp_root, "data") if exp_root else None)
    if base and "HF_HOME" not in os.environ:
        os.environ["HF_HOME"] = os.path.join(base, "huggingface")
