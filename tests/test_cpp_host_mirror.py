"""The C++ host mirror (include/kore_b200.hpp): compiles against the C ABI on any machine;
on a GPU its test program checks the CUDA path against the CPU restatement."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
OUT_DIR = os.path.join(ROOT, "tests", "cpp", "_build")
EXE = os.path.join(OUT_DIR, "host_mirror_test")


def _build():
    from kore_b200 import _build as kb_build
    from oracle import kbref

    lib = kb_build.build()
    ref = kbref.build()
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "oracle"), SRC,
           "-o", EXE, lib, ref, f"-Wl,-rpath,{os.path.dirname(lib)}", f"-Wl,-rpath,{os.path.dirname(ref)}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return EXE


def test_host_mirror_compiles_and_links():
    assert os.path.exists(_build())


@pytest.mark.gpu
def test_host_mirror_against_restatement():
    exe = _build()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip().startswith("OK ")
