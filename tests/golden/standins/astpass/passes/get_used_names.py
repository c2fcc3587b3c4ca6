"""analyze(tree, no_funcname=True): names in order of first use, callee names left out
(how appy/dispatcher.py:14 uses it)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
    os.path.dirname(os.path.abspath(__file__))))))))
from appy_b200.frontend.loop_normalize import used_names  # noqa: E402


def analyze(tree, no_funcname=True):
    return used_names(tree)
