"""A plain C++ program (tests/native/drop_in.cpp) built against include/NativeOps.h and linked to the shared
library calls the exported, mangled NativeOps members with the reference's CUDA-build conventions (device
shapeInfo and dimension arrays, host copies and the stream in extraPointers). This is the path nd4j's JNI
glue takes; the other GPU tests enter through the C ABI."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_caller_through_the_mangled_members(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++ on this machine")
    libdir = os.path.join(ROOT, "libnd4j_b200")
    exe = str(tmp_path / "drop_in")
    subprocess.run([gxx, "-std=c++11", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "native", "drop_in.cpp"),
                    "-L", libdir, "-lnd4jb200", "-Wl,-rpath," + libdir, "-o", exe], check=True)
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "drop-in ok" in run.stdout
