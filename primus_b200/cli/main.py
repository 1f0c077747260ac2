"""``primus`` command line: ``primus {train,benchmark,preflight,node_smoke,projection,data} ...``.

Sub-commands are plug-ins: every module in ``primus_b200/cli/subcommands`` that defines
``register_subcommand(subparsers)`` and sets ``func`` via ``set_defaults`` is discovered with
``pkgutil``; only the requested one is imported.  Unknown arguments are forwarded to the
sub-commands that accept free-form overrides (train / projection / preflight).
(primus/cli/main.py:54-111,140-226 in the reference.)
"""
from __future__ import annotations

import argparse
import importlib
import os
import pkgutil
import sys
import traceback

FORWARD_UNKNOWN = {"train", "projection", "preflight"}


def discover_subcommands() -> list[str]:
    from . import subcommands

    return sorted(m.name for m in pkgutil.iter_modules(subcommands.__path__) if not m.name.startswith("_"))


def build_parser(only: str | None = None) -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="primus", description="primus-b200: Blackwell-native LLM training framework")
    parser.add_argument("--debug", action="store_true", help="set PRIMUS_LOG_LEVEL=DEBUG")
    parser.add_argument("--version", action="store_true")
    sub = parser.add_subparsers(dest="command")
    for name in discover_subcommands():
        if only and name != only:
            sub.add_parser(name, help=f"{name} (not loaded)", add_help=False)
            continue
        mod = importlib.import_module(f"{__package__}.subcommands.{name}")
        if hasattr(mod, "register_subcommand"):
            mod.register_subcommand(sub)
    return parser


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    requested = next((a for a in argv if not a.startswith("-")), None)
    names = discover_subcommands()
    parser = build_parser(requested if requested in names else None)
    args, unknown = parser.parse_known_args(argv)
    if args.version:
        from .. import __version__

        print(__version__)
        return 0
    if args.debug:
        os.environ["PRIMUS_LOG_LEVEL"] = "DEBUG"
    if not getattr(args, "command", None) or not hasattr(args, "func"):
        parser.print_help()
        return 1
    if unknown and args.command not in FORWARD_UNKNOWN:
        parser.error(f"unrecognized arguments: {' '.join(unknown)}")
    try:
        rc = args.func(args, unknown)
        return int(rc or 0)
    except KeyboardInterrupt:
        return 130
    except Exception as e:  # noqa: BLE001
        tb = traceback.extract_tb(e.__traceback__)
        last = tb[-1] if tb else None
        where = f" ({os.path.basename(last.filename)}:{last.lineno} in {last.name})" if last else ""
        print(f"[primus] {args.command} failed: {type(e).__name__}: {e}{where}", file=sys.stderr)
        if os.environ.get("PRIMUS_LOG_LEVEL", "").upper() == "DEBUG":
            traceback.print_exc()
        return 1


if __name__ == "__main__":
    if not __package__:
        # started as a script (`torchrun primus_b200/cli/main.py ...`, the way the launcher starts the workers): run the
        # module of the same name inside its package so that the relative imports resolve
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        from primus_b200.cli.main import main as _package_main

        sys.exit(_package_main())
    sys.exit(main())
