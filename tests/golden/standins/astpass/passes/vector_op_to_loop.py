"""transform(tree, rt_vals): 1-D slice statements -> explicit loops tagged ``_simd_okay`` and
``_reduction=(op, var)``, the contract appy/backends/triton/passes/lower_array_op_to_loop.py:5-22
relies on.  The lowering itself is appy_b200's (the real package's source is not available), so
results that depend on it are NOT pinned to the reference."""
import ast
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
    os.path.dirname(os.path.abspath(__file__))))))))
from appy_b200.frontend.loop_normalize import SliceLowering  # noqa: E402


def transform(tree, rt_vals):
    low = SliceLowering(lambda name: getattr(rt_vals.get(name), "ndim", None))
    for node in ast.walk(tree):
        if isinstance(node, ast.For) and hasattr(node, "pragma") and "parallel_for" in node.pragma:
            node.body = low.lower_block(node.body)
    for node in ast.walk(tree):
        if isinstance(node, ast.For) and getattr(node, "_from_slice", False):
            red = node.pragma.get("reduction")
            del node.pragma
            node._simd_okay = True
            if red:
                op, var = red.split(":", 1)
                node._reduction = ("sum" if op == "+" else op, var)
    # extents of full slices are runtime shapes: inline them as constants
    import re

    class Inline(ast.NodeTransformer):
        def visit_Name(self, node):
            m = re.fullmatch(r"(\w+?)_shape_(\d+)", node.id)
            if m and node.id not in rt_vals and m.group(1) in rt_vals and hasattr(rt_vals[m.group(1)], "shape"):
                return ast.Constant(int(rt_vals[m.group(1)].shape[int(m.group(2))]))
            return node

    tree = Inline().visit(tree)
    ast.fix_missing_locations(tree)
    return tree
