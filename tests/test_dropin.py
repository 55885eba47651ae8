"""The library as a drop-in for the exocc-generated C: callers written like the
reference's own C / C++ harnesses (tests/dropin/), compiled with gcc / g++
against include/exo_b200.h and linked with libexo_b200.so -- no Python between
the caller and the C ABI."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "dropin")
LIBDIR = os.path.join(ROOT, "exo_b200")


def build(tmp_path, name, compiler, extra=()):
    from exo_b200 import build as b

    b.build()
    exe = tmp_path / name.split(".")[0]
    subprocess.run([compiler, "-O2", *extra, "-I", os.path.join(ROOT, "include"), os.path.join(SRC, name),
                    "-o", str(exe), "-L", LIBDIR, "-lexo_b200", f"-Wl,-rpath,{LIBDIR}", "-lm"], check=True)
    return str(exe)


def test_harnesses_compile_and_link(tmp_path):
    """CPU-only part: the C and C++ callers compile against the header and link."""
    build(tmp_path, "sgemm_check.cpp", "g++", ["-std=c++17"])
    build(tmp_path, "matmul_check.c", "gcc", ["-std=gnu11"])
    build(tmp_path, "conv_check.cpp", "g++", ["-std=c++17"])
    build(tmp_path, "shim_check.c", "gcc", ["-std=gnu11"])


@pytest.mark.gpu
def test_gemmini_shim_c_caller(tmp_path):
    """tiled_matmul_auto / tiled_conv_auto with the upstream parameter lists: generated
    instances, generic shapes, and refused requests."""
    exe = build(tmp_path, "shim_check.c", "gcc", ["-std=gnu11"])
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Correct" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(100, 100, 100), (1000, 1000, 1000), (37, 515, 129)])
def test_sgemm_cpp_caller(tmp_path, shape):
    exe = build(tmp_path, "sgemm_check.cpp", "g++", ["-std=c++17"])
    r = subprocess.run([exe, *map(str, shape)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().startswith("0 mismatches")


@pytest.mark.gpu
def test_gemmini_c_caller(tmp_path):
    exe = build(tmp_path, "matmul_check.c", "gcc", ["-std=gnu11"])
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Correct" in r.stdout


@pytest.mark.gpu
def test_conv_cpp_caller(tmp_path):
    exe = build(tmp_path, "conv_check.cpp", "g++", ["-std=c++17"])
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().startswith("0 mismatches")
