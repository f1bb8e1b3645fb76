"""The C++ call surface at run time: a program written against the reference's header paths,
class names and call sequence (tests/cpp/block_sequence_test.cpp) is compiled with g++ against
csrc/compat, linked to the library and run on the GPU."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_block_call_sequence_through_the_cpp_surface(tmp_path):
    from f2k_cuda_b200.build import LIB_PATH, build
    build()
    exe = tmp_path / "block_sequence_test"
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-I", str(ROOT / "f2k_cuda_b200/csrc/compat"),
           "-I", "/usr/local/cuda/include", str(ROOT / "tests/cpp/block_sequence_test.cpp"), "-o", str(exe),
           str(LIB_PATH), f"-Wl,-rpath,{LIB_PATH.parent}", "-L/usr/local/cuda/lib64", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PASS") == 3 and "FAIL" not in r.stdout, r.stdout
