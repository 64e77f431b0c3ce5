"""The C++ mirror of the reference's API (include/peregrine_b200.hpp): compiles on the CPU box, and on
a B200 runs the reference's own quant/gguf tests (tests/cpp/reference_tests.cpp) through it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "reference_tests")


def _build():
    from peregrine_b200.build import ensure_built

    lib = ensure_built()
    libdir = os.path.dirname(lib)
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "reference_tests.cpp"),
           "-o", EXE, "-L", libdir, "-lperegrine_b200", f"-Wl,-rpath,{libdir}"]
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.run(cmd, check=True, capture_output=True, text=True, env=env)


def test_cpp_mirror_compiles_and_links():
    _build()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_reference_tests_through_cpp_mirror():
    _build()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all reference tests passed" in r.stdout
