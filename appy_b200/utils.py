"""Pragma text <-> dict conversion and code dumping.

Mirrors the observable behaviour of the reference helpers (appy/utils.py:82-172):
``#pragma parallel for simd shared(a, b)`` becomes an ordered dict with the keys
``parallel_for``, ``simd``, ``shared`` ...; an unknown clause raises ``ValueError``
naming the clause (tested by tests/unit/general/pragma/test_invalid_pragma.py).
"""
from __future__ import annotations

import re
from collections import OrderedDict

RECOGNIZED_CLAUSES = ("parallel_for", "simd", "block", "reduction", "shared", "to", "from", "atomic")
_LIST_CLAUSES = ("shared", "to", "from")
_CLAUSE_RE = re.compile(r"(\w+)\s*\(([^)]*)\)")
_WORD_RE = re.compile(r"\w+")


def is_pragma(text) -> bool:
    return isinstance(text, str) and text.lstrip().startswith("#pragma")


def parse_pragma(pragma_str: str) -> "OrderedDict[str, object]":
    text = pragma_str.strip()
    if text.startswith("#"):
        text = text[1:].lstrip()
    if text.startswith("pragma"):
        text = text[len("pragma"):]
    text = text.strip()
    tokens: list[tuple[str, object]] = []
    pos = 0
    while pos < len(text):
        if text[pos].isspace():
            pos += 1
            continue
        m = _CLAUSE_RE.match(text, pos)
        if m:
            key = m.group(1)
            vals = tuple(v.strip() for v in m.group(2).split(",") if v.strip())
            if key in _LIST_CLAUSES:
                tokens.append((key, list(vals)))
            else:
                tokens.append((key, vals if len(vals) != 1 else vals[0]))
            pos = m.end()
            continue
        m = _WORD_RE.match(text, pos)
        if not m:
            raise ValueError(f"Unexpected syntax at: {text[pos:]}")
        tokens.append((m.group(0), True))
        pos = m.end()
    out: "OrderedDict[str, object]" = OrderedDict()
    skip = False
    for n, (key, val) in enumerate(tokens):
        if skip:
            skip = False
            continue
        if key == "parallel" and n + 1 < len(tokens) and tokens[n + 1][0] == "for":
            out["parallel_for"] = True
            skip = True
        else:
            out[key] = val
    for key in out:
        if key not in RECOGNIZED_CLAUSES:
            raise ValueError(f"Unrecognized pragma clause: `{key}` in `{text}`")
    return out


def dict_to_pragma(pragma: dict) -> str:
    words = []
    if pragma.get("parallel_for"):
        words += ["parallel", "for"]
    for key, val in pragma.items():
        if key == "parallel_for":
            continue
        if val is True:
            words.append(key)
        elif isinstance(val, (tuple, list)):
            words.append(f"{key}({', '.join(val)})")
        else:
            words.append(f"{key}({val})")
    return "#pragma " + " ".join(words)


def pretty_dump(src: str, loop_name: str) -> None:
    print(f"--- Dumped code for loop {loop_name} ---")
    print(src)
    print(f"--- End of dumped code for loop {loop_name} ---")
