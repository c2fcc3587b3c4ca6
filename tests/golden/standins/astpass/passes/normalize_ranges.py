import ast


def transform(tree):
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == "range":
            if len(node.args) == 1:
                node.args = [ast.Constant(0), node.args[0], ast.Constant(1)]
            elif len(node.args) == 2:
                node.args = [node.args[0], node.args[1], ast.Constant(1)]
    return tree
