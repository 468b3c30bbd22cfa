"""The C-ABI library loads and exports every symbol include/b200p.h declares;
argument errors are reported before any launch.  No GPU, no compute."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    """Every function any include/*.h declares."""
    import glob
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names |= set(re.findall(r"\b(b200p_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_what_python_binds(b200p):
    assert header_symbols() == sorted(b200p.SYMBOLS)


def test_library_exports_every_declared_symbol(b200p):
    h = C.CDLL(b200p.LIB_PATH)
    for name in header_symbols():
        assert hasattr(h, name), name
    assert b"sm_100a" in b200p.lib().b200p_version()


def test_argument_errors_come_before_any_launch(b200p):
    L = b200p.lib()
    n0 = b200p.launch_count()
    assert L.b200p_segreduce(b200p.SUM, 99, None, None, 64, None) == -2          # dtype
    assert L.b200p_segreduce(7, b200p.F32, None, None, 64, None) == -3           # op
    assert L.b200p_segreduce(b200p.SUM, b200p.F32, None, None, 63, None) == -4   # length
    assert L.b200p_segreduce(b200p.SUM, b200p.F32, None, None, 64, None) == -1   # null
    assert L.b200p_segreduce(b200p.SUM, b200p.F32, None, None, 0, None) == 0     # empty input: nothing to do
    assert L.b200p_segscan_inclusive(b200p.SUM, b200p.F32, None, None, 128, None) == -1
    assert L.b200p_segscan_exclusive_sum(b200p.F16, None, None, 64, None) == -2
    assert L.b200p_segreduce_narrow(b200p.SUM, b200p.F32, None, None, 64, None) == -2
    assert L.b200p_wave_probe(5, 0, 0, None, None, None) == -3
    assert b200p.launch_count() == n0
    assert b200p.lib().b200p_strerror(-4).decode().startswith("length")
    assert b200p.set_tuning("no_such_knob", 1) == -2 ** 31


def test_no_cpu_fallback(b200p):
    import torch
    x = torch.zeros(64)
    with pytest.raises(ValueError):
        b200p.segreduce(x)


def test_cpp_api_header_compiles_and_links(b200p, tmp_path):
    """include/cdna3/attention.hpp (the reference-shaped C++ API) builds with g++ alone and
    links against the C-ABI library; argument errors come back without touching a GPU."""
    import subprocess
    exe = tmp_path / "api_compile"
    lib_dir = os.path.dirname(b200p.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                    os.path.join(ROOT, "tests", "cpp", "api_compile.cpp"), "-L" + lib_dir, "-lb200p",
                    "-Wl,-rpath," + lib_dir, "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
