"""The C++ facade (vq_b200/cpp/vq.hpp) compiled and run against the reference's own test cases."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_facade.cpp")
LIBDIR = os.path.join(ROOT, "vq_b200")


def _build(out):
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-o", out, SRC, "-L" + LIBDIR, "-lvqb",
                           "-Wl,-rpath," + LIBDIR])


def test_facade_compiles_and_links(tmp_path):
    """No GPU needed: the header is valid C++17 and every entry point it uses exists in libvqb.so."""
    _build(os.path.join(str(tmp_path), "test_facade"))


@pytest.mark.gpu
def test_reference_tests_through_the_cpp_facade(tmp_path):
    exe = os.path.join(str(tmp_path), "test_facade")
    _build(exe)
    res = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=600)
    out = res.stdout.decode()
    assert res.returncode == 0 and "all facade checks passed" in out, out[-3000:]
