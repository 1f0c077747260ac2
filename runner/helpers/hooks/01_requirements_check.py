#!/usr/bin/env python3
"""Global hook: check that the Python side can run (torch with CUDA 12.8+, numpy, yaml) and say what is missing.
Warnings go to stderr through the hook protocol (any line that is not env.* / extra.* is passed through); a missing
hard requirement fails the launch unless PRIMUS_SKIP_REQUIREMENTS_CHECK=1."""
import importlib
import os
import sys

if os.environ.get("PRIMUS_SKIP_REQUIREMENTS_CHECK", "0") == "1":
    sys.exit(0)
hard, soft = ["torch", "numpy", "yaml"], ["tabulate", "sentencepiece", "transformers", "tensorboard"]
missing = [m for m in hard if importlib.util.find_spec(m) is None]
if missing:
    print("missing required python packages: " + ", ".join(missing))
    sys.exit(0 if os.environ.get("PRIMUS_DRY_RUN", "0") == "1" else 2)
for m in soft:
    if importlib.util.find_spec(m) is None:
        print(f"optional python package not found: {m}")
import torch  # noqa: E402

cuda = torch.version.cuda or ""
if cuda and tuple(int(x) for x in cuda.split(".")[:2]) < (12, 8):
    print(f"torch was built for CUDA {cuda}; sm_100a kernels need a 12.8+ runtime")
print(f"env.PRIMUS_TORCH_VERSION={torch.__version__}")
