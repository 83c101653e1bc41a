"""The C++ operator API (include/slopfab_b200/linear.hpp) compiles, links and -- on a GPU -- reproduces the
reference's W4A8 known-answer test when used exactly like the reference's LinearRunner."""
import os
import subprocess

import numpy as np
import pytest

import oracle
import slopfab_b200 as sfq
from test_oracle_golden import _packed_case

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "drop_in")


def _build():
    src = os.path.join(ROOT, "tests", "cpp", "drop_in.cu")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(sfq.LIB_PATH)):
        subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"),
                        src, "-o", EXE, "-L", os.path.dirname(sfq.LIB_PATH), "-lsfq", "-Xlinker", "-rpath",
                        "-Xlinker", os.path.dirname(sfq.LIB_PATH)], check=True, capture_output=True)


def test_cpp_api_compiles_and_links():
    _build()
    out = subprocess.run([EXE, "link-only"], capture_output=True, text=True)
    assert out.returncode == 0 and "linked" in out.stdout, out.stderr


@pytest.mark.gpu
def test_cpp_api_runs_the_reference_known_answer():
    _build()
    out = subprocess.run([EXE], capture_output=True, text=True)
    assert out.returncode == 0, (out.returncode, out.stderr)
    got = np.array([int(v) for v in out.stdout.split()], np.uint16).reshape(3, 4)
    packed, levels, scales, book, channel, x = _packed_case(4, 16)
    want = oracle.packed_int8_linear(oracle.to_bf16(x), packed, scales, channel, book, 4, 16, 4, 256)
    assert np.array_equal(got, want)
