"""``primus node_smoke``: single-process acceptance test of one node — inventory, native-library check and, on
every local GPU in turn, a tiny training step through the sm_100a kernels plus the tier-2 performance checks
(primus/tools/preflight/node_smoke/* in the reference; the launcher runs it with ``--single``)."""
from __future__ import annotations

import json


def register_subcommand(subparsers):
    p = subparsers.add_parser("node_smoke", help="per-node smoke test")
    p.add_argument("--no-perf", action="store_true")
    p.add_argument("--json", action="store_true")
    p.set_defaults(func=run)


def run(args, unknown):
    import torch

    from ...tools.preflight.checks import run_preflight

    rep = run_preflight(perf=not args.no_perf)
    if torch.cuda.is_available() and rep["native"]["present"]:
        from ...engine.trainer import TrainConfig, Trainer
        from ...models.config import TransformerConfig
        from ...ops import _lib
        from ...parallel import state as ps

        for d in range(torch.cuda.device_count()):
            try:
                torch.cuda.set_device(d)
                ps.destroy_model_parallel()
                cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1408, num_attention_heads=4,
                                        num_query_groups=2, kv_channels=128, vocab_size=32000, params_dtype="bf16")
                tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=2, log_interval=1)
                losses = Trainer(cfg, tc, device=f"cuda:{d}", log_fn=lambda s: None).train(2)
                torch.cuda.synchronize()
                _lib.check_status(d)
                ok = all(l == l for l in losses)
                rep["checks"].append({"check": f"training step on GPU {d}", "status": "PASS" if ok else "FAIL",
                                      "detail": f"losses {losses}"})
            except Exception as e:  # noqa: BLE001
                rep["checks"].append({"check": f"training step on GPU {d}", "status": "FAIL", "detail": repr(e)})
    if args.json:
        print(json.dumps(rep, indent=1, default=str))
    else:
        for c in rep["checks"]:
            print(f"  [{c['status']}] {c['check']}: {c['detail']}")
    return 1 if any(c["status"] == "FAIL" for c in rep["checks"]) else 0
