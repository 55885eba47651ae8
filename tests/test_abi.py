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
SHIM_HEADER = os.path.join(ROOT, "include", "exo_b200_gemmini_shim.h")
PROTOTYPES = os.path.join(ROOT, "tests", "golden", "generated_prototypes.txt")


@pytest.fixture(scope="module")
def built():
    from exo_b200 import build

    return build.build()


def declared_symbols(headers=(HEADER, SHIM_HEADER)):
    out = set()
    for h in headers:
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
        text = re.sub(r"\s+", " ", text)  # the shim's prototypes span several lines
        for stmt in text.split(";"):
            m = re.search(r"\b(\w+) ?\(", stmt)
            if m and "typedef" not in stmt[:m.start()]:
                out.add(m.group(1))
    return sorted(out - {"defined", "push", "visibility"})


def test_header_repeats_the_generated_prototypes_token_for_token():
    """Every public prototype exocc wrote into the generated headers of the three apps
    (tests/golden/generated_prototypes.txt, extracted from the reference's golden files by
    tests/golden/make_prototypes.py) appears in include/exo_b200.h as the same line, once
    the context type macro is set to the generated header's own type."""
    # expand the one macro by hand (the preprocessor would also rewrite bool to _Bool)
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    lines = {l.strip().replace("EXO_B200_GEMMINI_CONTEXT", "test_case_Context") for l in text.splitlines()}
    want = [l.split(": ", 1)[1].strip() for l in open(PROTOTYPES).read().splitlines() if l.strip()]
    assert len(want) == 20
    missing = [w for w in want if w not in lines]
    assert not missing, missing
    # and with the default (void) the same header still declares sgemm_exo / conv_specialized verbatim
    text = open(HEADER).read()
    for w in want[:2]:
        assert w in text


def test_library_exports_every_declared_symbol(built):
    out = subprocess.run(["nm", "-D", "--defined-only", built], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    declared = declared_symbols()
    assert len(declared) >= 41 and "tiled_matmul_auto" in declared and "ssyrk_exo" in declared
    missing = [s for s in declared if s not in exported]
    assert not missing, missing
    # nothing but the declared C ABI leaks out of the library
    assert exported <= set(declared), sorted(exported - set(declared))


def test_ctypes_prototypes_cover_header(built):
    from exo_b200 import _lib

    declared = set(declared_symbols())
    assert declared == set(_lib.PROTOTYPES) | set(_lib.SUPPORT)


def test_header_coexists_with_a_generated_header(tmp_path):
    """A translation unit that includes a generated Gemmini header (its context struct and
    prototypes) and this header with the context type macro set compiles without conflicting
    declarations."""
    gen = tmp_path / "gemmini_lib.h"
    gen.write_text("#include <stdint.h>\n#include <stdbool.h>\n"
                   "typedef struct gemmini_lib_Context { struct { float scale; } ConfigLoad; } gemmini_lib_Context;\n"
                   "void cpu_matmul_4( gemmini_lib_Context *ctxt, const float* scale, bool act, const int8_t* A, "
                   "const int8_t* B, int8_t* C );\n"
                   "void conv_3( gemmini_lib_Context *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, "
                   "const int8_t* weights, bool act, const float* scale );\n")
    src = tmp_path / "both.c"
    src.write_text('#include "gemmini_lib.h"\n#define EXO_B200_GEMMINI_CONTEXT gemmini_lib_Context\n'
                   '#include "exo_b200.h"\n#include "exo_b200_gemmini_shim.h"\nint main(void){return 0;}\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(tmp_path), "-I", os.path.join(ROOT, "include"),
                    "-fsyntax-only", str(src)], check=True)


def test_header_compiles_as_c_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "exo_b200.h"\n#include "exo_b200_gemmini_shim.h"\nint main(void){return 0;}\n')
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


def test_sgemm_kernel_choice_is_pinned(built):
    """The exact SGEMM's dispatch (host logic, no GPU needed): the special kernels for few rows or columns and
    the tile configuration the measured cost table picks for the shapes it was fitted on.  A change of the
    table or of a threshold that moves one of these has to be a decision, not an accident."""
    import exo_b200

    f = exo_b200.library().dll.exo_b200_sgemm_kernel_choice
    tiles = lambda r, c: 1000000 + 1000 * r + c
    expected = {
        (32768, 8, 512): 1, (16384, 16, 512): 1, (1024, 16, 64): 1,          # tall kernel
        (1, 8192, 8192): 2, (2, 8192, 1024): 2,                              # TMA-fed GEMV
        (1, 8192, 300): 3, (3, 100, 100): 3, (4, 512, 300): 3, (1, 8193, 8192): 3,  # cp.async GEMV
        (8, 8192, 512): 4, (5, 16384, 1024): 4,                              # skinny kernel
        (8, 32768, 512): tiles(8, 128), (6, 65536, 256): tiles(8, 128),
        (16, 16384, 512): tiles(16, 64), (12, 1000, 700): tiles(32, 32), (17, 4099, 513): tiles(32, 32),
        (256, 256, 256): tiles(32, 32), (512, 512, 512): tiles(32, 32), (4096, 64, 4096): tiles(32, 32),
        (1024, 1024, 1024): tiles(128, 64), (1000, 1000, 1000): tiles(128, 64), (1536, 1536, 1536): tiles(128, 64),
        (1088, 1088, 1088): tiles(64, 64), (1280, 1280, 1280): tiles(64, 64),
        (2048, 2048, 2048): tiles(128, 128), (8192, 8192, 8192): tiles(128, 128),
    }
    got = {shape: f(*shape) for shape in expected}
    assert got == expected
    assert f(0, 4, 4) == -1 and f(4, 4, -1) == -1


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
