"""Stand-in for the third-party ``ast_comments`` package (not installed in this image),
used ONLY by tests/golden/make_golden.py to run the reference's own passes on CPU.

Behaviour provided: ``parse`` keeps stand-alone comment lines as ``Comment`` statement
nodes (``.value`` is the comment text, ``.inline`` False); ``unparse`` writes them back;
everything else is re-exported from ``ast``.  Written from the package's documented
behaviour; it is not a copy of its source.
"""
import ast as _ast
import io as _io
import tokenize as _tokenize
from ast import *  # noqa: F401,F403


class Comment(_ast.stmt):
    _fields = ("value", "inline")


_MARK = "__standin_comment__"


def parse(source, *args, **kwargs):
    lines = source.splitlines()
    try:
        toks = list(_tokenize.generate_tokens(_io.StringIO(source).readline))
    except (_tokenize.TokenError, IndentationError):
        toks = []
    for tok in toks:
        if tok.type == _tokenize.COMMENT and tok.line[: tok.start[1]].strip() == "":
            row, col = tok.start
            lines[row - 1] = lines[row - 1][:col] + f"{_MARK}({tok.string.rstrip()!r})"
    tree = _ast.parse("\n".join(lines) + "\n", *args, **kwargs)

    class Fix(_ast.NodeTransformer):
        def visit_Expr(self, node):
            v = node.value
            if isinstance(v, _ast.Call) and isinstance(v.func, _ast.Name) and v.func.id == _MARK:
                return _ast.copy_location(Comment(value=v.args[0].value, inline=False), node)
            return node

    return Fix().visit(tree)


class _Unparser(_ast._Unparser):
    def visit_Comment(self, node):
        self.fill(node.value)


def unparse(node):
    return _Unparser().visit(node)
