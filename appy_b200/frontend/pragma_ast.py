"""Parsing Python source while keeping ``#pragma`` comment lines.

The reference relies on the third-party ``ast_comments`` package to keep comments
as statement nodes (appy/__init__.py:40-41).  Here only pragma comments matter, so a
standalone ``#pragma ...`` line is turned, before parsing, into an expression
statement holding the pragma text as a string constant at the same indentation.
The ordinary ``ast`` module then parses and unparses everything; ``is_pragma_stmt``
recognises the markers and ``unparse`` turns them back into comment lines.
"""
from __future__ import annotations

import ast
import io
import tokenize


def _pragma_lines(source: str) -> dict[int, tuple[int, str]]:
    """line number -> (column, text) of comment tokens that stand alone on a line and
    start with ``#pragma``."""
    found: dict[int, tuple[int, str]] = {}
    try:
        toks = list(tokenize.generate_tokens(io.StringIO(source).readline))
    except (tokenize.TokenError, IndentationError):
        toks = []
    for tok in toks:
        if tok.type == tokenize.COMMENT and tok.string.startswith("#pragma"):
            line = tok.line
            if line[: tok.start[1]].strip() == "":
                found[tok.start[0]] = (tok.start[1], tok.string.rstrip())
    return found


def parse(source: str) -> ast.Module:
    marks = _pragma_lines(source)
    if marks:
        lines = source.splitlines()
        for lineno, (col, text) in marks.items():
            lines[lineno - 1] = lines[lineno - 1][:col] + repr(text)
        source = "\n".join(lines) + "\n"
    return ast.parse(source)


def pragma_text(node) -> str | None:
    """The pragma string if `node` is a pragma marker statement, else None."""
    if isinstance(node, ast.Expr) and isinstance(node.value, ast.Constant) \
            and isinstance(node.value.value, str) and node.value.value.startswith("#pragma"):
        return node.value.value
    return None


def unparse(tree) -> str:
    """``ast.unparse`` with pragma markers written back as comment lines."""
    out = []
    for line in ast.unparse(tree).splitlines():
        stripped = line.lstrip()
        if stripped[:1] in "'\"":
            try:
                val = ast.literal_eval(stripped)
            except (ValueError, SyntaxError):
                val = None
            if isinstance(val, str) and val.startswith("#pragma"):
                line = line[: len(line) - len(stripped)] + val
        out.append(line)
    return "\n".join(out)
