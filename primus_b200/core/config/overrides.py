"""Command-line overrides: ``key=value``, ``--key=value``, ``--key value``, bare ``--flag`` (true) and
dotted keys for nesting; values are coerced to bool / int / float / Python literals
(primus/core/utils/arg_utils.py:14-169 in the reference)."""
from __future__ import annotations

import ast
from typing import Any

from .merge import set_nested


def coerce_value(text: str) -> Any:
    low = text.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    try:
        return int(text)
    except ValueError:
        pass
    try:
        return float(text)
    except ValueError:
        pass
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        return text


def parse_cli_overrides(argv: list[str]) -> dict:
    out: dict = {}
    i = 0
    while i < len(argv):
        tok = argv[i]
        if tok.startswith("--"):
            body = tok[2:]
            if not body:
                raise ValueError("empty option '--'")
            if "=" in body:
                k, v = body.split("=", 1)
                set_nested(out, k, coerce_value(v))
            elif i + 1 < len(argv) and not argv[i + 1].startswith("--") and "=" not in argv[i + 1]:
                set_nested(out, body, coerce_value(argv[i + 1]))
                i += 1
            else:
                set_nested(out, body, True)
        elif "=" in tok:
            k, v = tok.split("=", 1)
            set_nested(out, k, coerce_value(v))
        else:
            raise ValueError(f"cannot parse override {tok!r}; use key=value or --key value")
        i += 1
    return out
