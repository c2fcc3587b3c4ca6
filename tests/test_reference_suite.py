"""The reference's own test files, run unmodified against this package.

Where a checkout of the reference is available (the APPY_REFERENCE_TREE environment variable,
or a directory named ``reference`` beside this repository), every test file under its
``tests/integration/triton`` and ``tests/unit/general`` trees is imported with ``appy``
resolving to this package and its test functions are executed.  No GPU is needed: the loops
run in ``dry_run`` mode (the dispatcher executes the plain loop, appy/dispatcher.py:46-53),
so the assertions of those files check the decoration-time rewrite (shape hoisting, shared
scalars, stubs, error messages), and every kernel the code generator produces for them is
compiled with NVRTC for sm_100a on the way.  The files are read where they lie; nothing of
them is stored in this repository.  Without a checkout the module is skipped.
"""
import glob
import importlib.util
import os
import re
import sys

import pytest

import appy_b200
from appy_b200.backends.cuda_sm100 import codegen as cg
from appy_b200.backends.cuda_sm100 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TREE = os.environ.get("APPY_REFERENCE_TREE") or os.path.join(os.path.dirname(ROOT), "reference")
FILES = sorted(
    p for p in glob.glob(os.path.join(TREE, "tests", "integration", "triton", "*", "*.py")) +
    glob.glob(os.path.join(TREE, "tests", "unit", "general", "**", "*.py"), recursive=True)
    if not os.path.basename(p).startswith("__"))

pytestmark = pytest.mark.skipif(not FILES, reason="no reference checkout on this machine")


@pytest.fixture()
def reference_view(monkeypatch):
    """`import appy` gives this package; loops default to dry_run; generated kernels are compiled."""
    compiled = []
    real_codegen = cg.codegen

    def codegen_and_compile(loop_source, loop_name, val_map, options):
        f, code_src = real_codegen(loop_source, loop_name, val_map, options)
        for variant in f.variants.values():
            plan = variant.plan
            if (plan.name, plan.source) in compiled:
                continue
            opts = [f"-D{k}={c[0]}" for k, c in plan.tunables.items()] + list(plan.info.get("nvrtc", []))
            rt.compile_check(plan.source, plan.name, opts)
            compiled.append((plan.name, plan.source))
        return f, code_src

    real_defaults = appy_b200.set_default_options

    def defaults_with_dry_run(options):
        real_defaults(options)
        options["dry_run"] = True

    from appy_b200 import dispatcher
    monkeypatch.setattr(cg, "codegen", codegen_and_compile)
    monkeypatch.setattr(dispatcher, "_sm100_codegen", codegen_and_compile)     # the dispatcher keeps its own reference
    monkeypatch.setattr(appy_b200, "set_default_options", defaults_with_dry_run)
    monkeypatch.setitem(sys.modules, "appy", appy_b200)
    return compiled


@pytest.mark.parametrize("path", FILES, ids=[os.path.relpath(p, TREE) for p in FILES])
def test_reference_test_file(path, reference_view):
    name = "reference_" + re.sub(r"\W", "_", os.path.relpath(path, TREE))
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    tests = [getattr(module, n) for n in sorted(dir(module)) if n.startswith("test") and callable(getattr(module, n))]
    assert tests, "the file defines no test function"
    for fn in tests:
        fn()
    wants_kernel = "irregular_range" not in path and "no_pragma" not in path
    assert reference_view or not wants_kernel, "no kernel was generated for this file"
