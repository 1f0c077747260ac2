"""Result tables of the benchmark and preflight tools as files: the format follows the file name
(``.md`` / ``.csv`` / ``.tsv`` / ``.jsonl``, each optionally ``.gz``), ``-`` or an empty name prints Markdown to the
terminal, and ``append`` adds rows to an existing file without repeating the header.  ``benchmark.common.emit`` routes its
``--output`` through this module for every extension other than ``.json``.

Counterpart of the reference's table writer (primus/tools/report.py ``write_table_simple``).
"""
from __future__ import annotations

import csv
import gzip
import io
import json
import os
from typing import Any, Optional, Sequence


def table_format(path: str) -> str:
    p = path.lower()
    if p.endswith(".gz"):
        p = p[:-3]
    for ext, fmt in ((".csv", "csv"), (".tsv", "tsv"), (".jsonl", "jsonl"), (".md", "md"), (".markdown", "md")):
        if p.endswith(ext):
            return fmt
    return "md"


def _markdown(header: Sequence[str], rows: Sequence[Sequence[Any]], with_header: bool) -> str:
    out = io.StringIO()
    if with_header:
        out.write("| " + " | ".join(str(h) for h in header) + " |\n")
        out.write("|" + "|".join("---" for _ in header) + "|\n")
    for r in rows:
        out.write("| " + " | ".join(str(x) for x in r) + " |\n")
    return out.getvalue()


def write_table(path: Optional[str], header: Sequence[str], rows: Sequence[Sequence[Any]], append: bool = False,
                preamble: Optional[str] = None) -> str:
    """Write (or append) a table; returns the text that was written."""
    if not path or path == "-":
        text = (preamble.rstrip("\n") + "\n\n" if preamble else "") + _markdown(header, rows, True)
        print(text, end="")
        return text
    fmt = table_format(path)
    exists = os.path.exists(path) and os.path.getsize(path) > 0
    fresh = not (append and exists)
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    buf = io.StringIO()
    if fmt == "md":
        if fresh and preamble:
            buf.write(preamble.rstrip("\n") + "\n\n")
        buf.write(_markdown(header, rows, fresh))
    elif fmt in ("csv", "tsv"):
        w = csv.writer(buf, delimiter="," if fmt == "csv" else "\t", lineterminator="\n")
        if fresh:
            w.writerow(header)
        w.writerows(rows)
    else:
        for r in rows:
            buf.write(json.dumps(dict(zip(header, r))) + "\n")
    text = buf.getvalue()
    opener = gzip.open if path.lower().endswith(".gz") else open
    with opener(path, "at" if not fresh else "wt") as f:
        f.write(text)
    return text


def write_records(path: Optional[str], records: Sequence[dict], append: bool = False, preamble: Optional[str] = None) -> str:
    """``write_table`` for a list of dicts (the union of the keys, in first-seen order, is the header)."""
    header: list = []
    for r in records:
        for k in r:
            if k not in header:
                header.append(k)
    return write_table(path, header, [[r.get(k, "") for k in header] for r in records], append, preamble)
