"""``primus train {pretrain,posttrain} --config exp.yaml [--export_config out.yaml] [overrides ...]``
(primus/cli/subcommands/train.py:12-78, primus/core/launcher/parser.py:18-53 in the reference)."""
from __future__ import annotations


def register_subcommand(subparsers):
    p = subparsers.add_parser("train", help="launch a training module")
    sp = p.add_subparsers(dest="suite", required=True)
    for name in ("pretrain", "posttrain"):
        q = sp.add_parser(name)
        q.add_argument("--config", "--exp", dest="config", required=True, help="experiment YAML")
        q.add_argument("--data_path", default=None)
        q.add_argument("--backend_path", default=None, help="accepted for compatibility; unused (single backend)")
        q.add_argument("--export_config", default=None, help="write the fully resolved config here")
        q.add_argument("--dry-run", dest="dry_run", action="store_true", help="resolve the config and exit")
    p.set_defaults(func=run)


def run(args, overrides):
    import os

    from ...core.runtime.train_runtime import PrimusRuntime

    if args.data_path:
        os.environ["DATA_PATH"] = args.data_path
    rt = PrimusRuntime(args.config, overrides, args.export_config)
    module = "pre_trainer" if args.suite == "pretrain" else "post_trainer"
    if args.dry_run:
        rt._initialize_configuration(module)
        import yaml

        print(yaml.safe_dump(rt.ctx.experiment.export(), sort_keys=False))
        return 0
    rt.run_train_module(module)
    return 0
