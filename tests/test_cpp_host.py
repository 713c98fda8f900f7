"""Builds and runs the C++ test executables of the host operator API
(cut_b200/csrc/host): the host-logic suite on the CPU with a recording backend,
and the reference's known-answer cases through Runtime/Operations on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "cut_b200", "csrc", "host")
CPP = os.path.join(ROOT, "tests", "cpp")
OUT = os.path.join(ROOT, "tests", "cpp", "build")


def _compile(args, exe):
    os.makedirs(OUT, exist_ok=True)
    r = subprocess.run(["g++", "-O1", "-std=c++17", f"-I{HOST}", f"-I{CPP}", "-o", exe, *args], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def _run(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failures" in r.stdout, r.stdout


def test_host_logic_cpu():
    exe = os.path.join(OUT, "host_logic_test")
    _compile([os.path.join(CPP, "host_logic_test.cpp"), os.path.join(HOST, "cut_api.cpp"), os.path.join(HOST, "gguf_upload.cpp")], exe)
    _run(exe)


def test_host_library_builds_and_links():
    """libcut_host.so (operator API + B200 backend) links against libcutb.so and exports the factory."""
    from cut_b200 import build as b

    lib = b.build_host()
    out = subprocess.run(["nm", "-DC", lib], capture_output=True, text=True).stdout
    assert "cut::createB200Compute(int)" in out
    assert "cut::Operations::matmul(" in out and "cut::VariantSelector::select(" in out


@pytest.mark.gpu
def test_reference_cases_through_operator_api_gpu():
    from cut_b200 import build as b
    from oracle import oracle as O

    b.build_host()
    O.lib()
    exe = os.path.join(OUT, "reference_cases_test")
    pkg = os.path.join(ROOT, "cut_b200")
    orc = os.path.join(ROOT, "oracle", "_build")
    _compile([os.path.join(CPP, "reference_cases_test.cpp"), f"-L{pkg}", "-lcut_host", "-lcutb", f"-L{orc}", "-loracle",
              f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{orc}"], exe)
    _run(exe)
