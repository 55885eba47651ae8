"""CPU-only checks of the drop-in boundary: the shared library loads, exports
every symbol that include/exo_b200.h declares, and reports errors through the
side channel instead of computing anything on the CPU."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "exo_b200.h")


@pytest.fixture(scope="module")
def built():
    from exo_b200 import build

    return build.build()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"^[\w\s\*]+?\b(\w+)\s*\(", text, flags=re.M)) - {"defined"})


def test_header_declares_reference_prototypes():
    text = open(HEADER).read()
    # character-for-character the prototypes exocc generates
    assert ("void sgemm_exo( void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, "
            "const float* A, const float* B, float* C );") in text
    assert ("void conv_specialized( void *ctxt, const float* inp, float* output, "
            "const float* weights, const float* bias );") in text
    assert "const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );" in text


def test_library_exports_every_declared_symbol(built):
    out = subprocess.run(["nm", "-D", "--defined-only", built], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    declared = declared_symbols()
    assert len(declared) >= 36
    missing = [s for s in declared if s not in exported]
    assert not missing, missing
    # nothing but the declared C ABI leaks out of the library
    assert exported <= set(declared), sorted(exported - set(declared))


def test_ctypes_prototypes_cover_header(built):
    from exo_b200 import _lib

    declared = set(declared_symbols())
    assert declared == set(_lib.PROTOTYPES) | set(_lib.SUPPORT)


def test_header_compiles_as_c_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "exo_b200.h"\nint main(void){return 0;}\n')
    for cc, std in (("gcc", "-std=c11"), ("g++", "-std=c++17")):
        subprocess.run([cc, std, "-x", "c" if cc == "gcc" else "c++", "-I", os.path.join(ROOT, "include"),
                        "-fsyntax-only", str(src)], check=True)


def test_size_type_is_64_bit(tmp_path):
    src = tmp_path / "s.c"
    src.write_text('#include <stdint.h>\n_Static_assert(sizeof(int_fast32_t) == 8, "int_fast32_t");\nint main(void){return 0;}\n')
    subprocess.run(["gcc", "-fsyntax-only", str(src)], check=True)


def test_invalid_arguments_are_reported_not_computed(built):
    import exo_b200

    lib = exo_b200.library()
    A = np.ones((4, 4), np.float32)
    C = np.zeros((4, 4), np.float32)
    with pytest.raises(exo_b200.ExoB200Error) as e:
        lib.sgemm_exo(None, 0, 4, 4, A, A, C)
    assert e.value.code == exo_b200.ERR_INVALID_ARGUMENT
    with pytest.raises(exo_b200.ExoB200Error) as e:
        lib.sgemm_exo(None, 4, 4, 4, A, None, C)
    assert e.value.code == exo_b200.ERR_INVALID_ARGUMENT
    with pytest.raises(exo_b200.ExoB200Error) as e:
        lib.conv(None, 3, 3, 4, 4, 4, 4, 3, 1, A, C, A, A)  # out_h != in_h - k + 1
    assert e.value.code == exo_b200.ERR_INVALID_ARGUMENT
    assert not C.any()


def test_no_cpu_fallback_without_a_device(built):
    """On a machine without a GPU a valid call must fail loudly, not compute."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import exo_b200

    lib = exo_b200.library()
    A = np.ones((4, 4), np.float32)
    C = np.zeros((4, 4), np.float32)
    with pytest.raises(exo_b200.ExoB200Error) as e:
        lib.sgemm_exo(None, 4, 4, 4, A, A, C)
    assert e.value.code in (exo_b200.ERR_CUDA, exo_b200.ERR_UNSUPPORTED)
    assert not C.any()


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "exo_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower().replace("oracle-free", ""), f
