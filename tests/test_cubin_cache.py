"""The on-disk cache of compiled kernels (appy_compile / appy_compile_image), exercised without a
GPU: an entry is found again, a truncated entry or one that carries another key is compiled afresh
and replaced instead of being loaded, a change to a template header changes the key, and the key is
the SHA-256 of what is documented (checked against hashlib)."""
import glob
import hashlib
import os
import shutil

from appy_b200.backends.cuda_sm100 import runtime as rt

SRC = 'extern "C" __global__ void k(float* a) { a[threadIdx.x] += 1.f; }'


def _entries(d):
    return sorted(glob.glob(os.path.join(d, "*.cubin")))


def test_entry_is_reused_and_a_damaged_one_is_replaced(tmp_path):
    d = str(tmp_path)
    n, hit = rt.compile_image(SRC, "k", [], d)
    assert n > 0 and not hit
    assert rt.compile_image(SRC, "k", [], d) == (n, True)
    (f,) = _entries(d)
    raw = open(f, "rb").read()
    assert raw.startswith(b"APPYCUBIN1\n" + os.path.basename(f)[:64].encode() + b"\n") and len(raw) > n
    # truncated file (a writer that died, a full disk)
    open(f, "wb").write(raw[: len(raw) // 2])
    assert rt.compile_image(SRC, "k", [], d) == (n, False)
    assert open(f, "rb").read() == raw                      # compiled afresh and written back whole
    # right name, but the header says the image belongs to another key
    open(f, "wb").write(raw[:11] + b"0" * 64 + raw[75:])
    assert rt.compile_image(SRC, "k", [], d) == (n, False)
    # a few bytes appended
    open(f, "wb").write(raw + b"xx")
    assert rt.compile_image(SRC, "k", [], d) == (n, False)
    assert rt.compile_image(SRC, "k", [], d) == (n, True)
    # other options, other entry
    assert rt.compile_image(SRC, "k", ["-DX=1"], d)[1] is False and len(_entries(d)) == 2


def _dir_digest(path):
    h = hashlib.sha256()
    for name in sorted(x for x in os.listdir(path) if not x.startswith(".")):
        with open(os.path.join(path, name), "rb") as fh:
            h.update(name.encode() + b"\x1f" + fh.read() + b"\x1e")
    return h.hexdigest()


def _expected_keys(src, opts):
    for major in (12, 13):
        for minor in range(10):
            h = hashlib.sha256()
            h.update(src.encode() + b"\x1f")
            for o in opts:
                h.update(o.encode() + b"\x1f")
                if o.startswith("-I"):
                    h.update(_dir_digest(o[2:]).encode())
            h.update(f"nvrtc {major}.{minor} sm_100a".encode())
            yield h.hexdigest()


def test_key_is_sha256_of_source_options_headers_compiler_and_target(tmp_path):
    d = str(tmp_path)
    rt.compile_image(SRC, "k", ["-DY=2"], d)
    (f,) = _entries(d)
    opts = ["--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "-I" + rt.template_dir(), "-DY=2"]
    assert os.path.basename(f)[:64] in set(_expected_keys(SRC, opts))


_CHILD = """
import sys
sys.path.insert(0, {root!r})
from appy_b200.backends.cuda_sm100 import runtime as rt
rt.template_dir = lambda: {inc!r}
print(rt.compile_image({src!r}, "k", [], {cache!r})[1])
"""


def test_a_changed_template_header_changes_the_key(tmp_path):
    """Generated sources only say `#include "t_flat.cuh"`: a fix to a header must not be served the
    cubin that was compiled before it.  Same directory, same source, same options; one process each
    (a process reads the headers once)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inc = tmp_path / "templates"
    shutil.copytree(rt.template_dir(), inc)
    cache = tmp_path / "cache"
    cache.mkdir()
    src = '#include "appy_device.cuh"\n' + SRC
    code = _CHILD.format(root=root, inc=str(inc), src=src, cache=str(cache))

    def child():
        res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stderr[-2000:]
        return res.stdout.strip().splitlines()[-1]

    assert child() == "False"
    assert child() == "True"
    with open(inc / "appy_device.cuh", "a") as fh:
        fh.write("\n// a fix\n")
    assert child() == "False"                           # not served from the old entry
    assert len(_entries(str(cache))) == 2
