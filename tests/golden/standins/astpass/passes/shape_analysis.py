"""analyze(tree, val_map) -> mapping from expression node to shape tuple, as consulted by
appy/backends/triton/passes/rewrite_vector_dot.py:33 for the operands of ``@``."""
import ast


class _Shapes(dict):
    def __init__(self, val_map):
        super().__init__()
        self.val_map = val_map

    def __missing__(self, node):
        if isinstance(node, ast.Name):
            return tuple(getattr(self.val_map.get(node.id), "shape", ()))
        if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name):
            base = tuple(getattr(self.val_map.get(node.value.id), "shape", ()))
            elts = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
            return tuple(base[d] for d, e in enumerate(elts) if isinstance(e, ast.Slice))
        return ()


def analyze(tree, val_map):
    return _Shapes(val_map)
