"""The C-ABI library builds, loads without a GPU, and exports every symbol that
include/appy_sm100.h declares (no compute calls here)."""
import os
import re

from appy_b200.backends.cuda_sm100 import runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "appy_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(appy_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "appy_compile" in syms and "appy_launch" in syms and "appy_spmm_csr_f32" in syms


def test_library_exports_every_declared_symbol():
    lib = runtime.lib()
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_table_matches_header():
    assert sorted(runtime.SIGNATURES) == declared_symbols()


def test_partition_range_host_logic():
    b = runtime.partition_range(0, 1000, 4, 32)
    assert b[0] == 0 and b[-1] == 1000 and all(x <= y for x, y in zip(b, b[1:]))
    assert all(x % 32 == 0 for x in b[1:-1])
    assert runtime.partition_range(5, 5, 3, 4) == [5, 5, 5, 5]
    b = runtime.partition_range(3, 10, 8, 1)
    assert b[0] == 3 and b[-1] == 10 and sum(y - x for x, y in zip(b, b[1:])) == 7


def test_partition_rows_balances_nonzeros():
    import numpy as np
    rng = np.random.default_rng(0)
    lens = rng.zipf(2.0, 20000).clip(max=500)
    indptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for parts in (1, 2, 3, 8):
        b = runtime.partition_rows(indptr, parts)
        assert b[0] == 0 and b[-1] == 20000 and all(x <= y for x, y in zip(b, b[1:]))
        per = [int(indptr[y] - indptr[x]) for x, y in zip(b, b[1:])]
        assert max(per) - min(per) <= 2 * 500
    b64 = runtime.partition_rows(indptr.astype(np.int64), 4)
    assert b64 == runtime.partition_rows(indptr, 4)
    # with a cost per row the ranges balance non-zeros + cost * rows: a range of short rows gets fewer rows
    lens = np.concatenate([np.full(9000, 2), np.full(1000, 200)])
    ip = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for cost in (0, 8, 100):
        b = runtime.partition_rows(ip, 4, cost)
        assert b[0] == 0 and b[-1] == 10000 and all(x <= y for x, y in zip(b, b[1:]))
        load = [int(ip[b[k + 1]] - ip[b[k]]) + cost * (b[k + 1] - b[k]) for k in range(4)]
        assert max(load) - min(load) <= 200 + cost
    assert runtime.partition_rows(ip, 4, 100)[1] < runtime.partition_rows(ip, 4, 0)[1]
