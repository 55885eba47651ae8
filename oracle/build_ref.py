"""TEST INFRASTRUCTURE -- never imported by the product package.

Builds the reference's own CPU implementation of the hot path into
``oracle/_ref/libexo_ref.so``.

Exo cannot be imported without its SMT dependencies, but the exact text that
``exocc`` generates for the three hot-path apps is checked into the reference
as golden test output (``tests/test_apps.py:13-33`` asserts byte equality of
``<header>\\n<c file>`` with ``tests/golden/test_apps/*.txt``).  This script
splits those files where they lie in the reference checkout, writes the pieces
to ``oracle/_ref/`` (git-ignored; reference sources are never committed) and
compiles them with gcc in GNU mode, i.e. with the default
``-ffp-contract=fast`` that the reference's own CMake build uses
(``tests/conftest.py:249-259`` sets no C standard), which matters for the
scalar corner loop of ``sgemm_above_kernel``.

What is taken from each golden:

* ``test_x86_sgemm.txt``   -> ``sgemm_exo``              (whole file)
* ``test_x86_conv.txt``    -> ``conv_specialized``       (whole file)
* ``test_gemmini_matmul.txt`` -> ``_relu_int8_t``, ``_select_float``,
  ``clamp`` and every ``cpu_matmul_*`` (the accelerator instruction streams
  ``matmul_*`` need a RISC-V toolchain and are left out)
* ``test_gemmini_conv.txt`` -> every ``conv_*_cpu``

The int8 files include ``<include/gemmini.h>`` from the un-vendored third-party
module ``exo-lang/gemmini-rocc-tests`` (pinned ``GIT_TAG exo-v3`` in
``apps/gemmini/CMakeLists.txt:35-44``).  Only one macro of it is used by the
CPU functions, ``ACC_SCALE``.  A one-line stub supplies it as round-half-even of
the fp32 product, the meaning this project's specification fixes
(``clamp(round_half_even(acc * acc_scale), -128, 127)``) and which the in-tree
sibling macro ``MVIN_SCALE_ACC`` = ``ROUND_NEAR_EVEN(x * scale)``
(``apps/gemmini/test/bare-metal/shims/include/gemmini_params.h.in:6-8``)
corroborates.  The reference's own tests never exercise a fractional scale, so
the rounding mode is pinned by the specification, not by the reference.

Usage:  python oracle/build_ref.py [--reference /path/to/exo]
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# Where the exo-lang/exo checkout lives: $EXO_REFERENCE, else a "reference" directory
# beside this repository.
DEFAULT_REFERENCE = os.environ.get(
    "EXO_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))

SPLIT_MARK = '#include "test_case.h"'

GEMMINI_STUB = """\
#pragma once
/* Stub for the un-vendored gemmini-rocc-tests header: only ACC_SCALE is needed
 * by the cpu_* functions.  Round-half-even of the fp32 product. */
#include <math.h>
#define ACC_SCALE(x, scale) (nearbyintf((float)(x) * (scale)))
"""


def _split(path: str) -> tuple[str, str]:
    text = open(path).read()
    idx = text.index(SPLIT_MARK)
    return text[:idx], text[idx:]


def _extract_function(c_text: str, signature_re: str) -> str:
    """Return the definition (signature line through matching brace)."""
    m = re.search(signature_re, c_text, flags=re.M)
    if m is None:
        raise RuntimeError(f"pattern not found: {signature_re}")
    start = m.start()
    i = c_text.index("{", m.end() - 1)
    depth = 0
    while True:
        ch = c_text[i]
        if ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0:
                return c_text[start : i + 1] + "\n"
        i += 1


def _write(rel: str, text: str) -> str:
    path = os.path.join(OUT, rel)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        f.write(text)
    return path


def _int8_unit(golden: str, stem: str, fn_re: str) -> str:
    header, c_text = _split(golden)
    header = header.replace("TEST_CASE_H", f"TEST_CASE_{stem.upper()}_H")
    names = sorted(set(re.findall(fn_re, c_text, flags=re.M)))
    body = [f'#include "test_case.h"\n#include <include/gemmini.h>\n']
    # The two extern helpers are emitted as non-static globals by exocc; make
    # them static here so the two int8 units can share one shared object.
    body.append("static " + _extract_function(c_text, r"^int8_t _relu_int8_t\(int8_t x\) \{"))
    body.append("static " + _extract_function(c_text, r"^float _select_float\(float x,float v,float y,float z\) \{"))
    body.append(_extract_function(c_text, r"^static void clamp\( [^;]*\) \{"))
    for n in names:
        body.append(_extract_function(c_text, rf"^void {n}\( [^;]*\) \{{"))
    _write(f"{stem}/test_case.h", header)
    _write(f"{stem}/include/gemmini.h", GEMMINI_STUB)
    return _write(f"{stem}/{stem}.c", "\n".join(body))


def build(reference: str = DEFAULT_REFERENCE, verbose: bool = True) -> str | None:
    """Extract + compile.  Returns the .so path, or None when the reference
    checkout (or AVX-512 gcc support) is not available."""
    golden = os.path.join(reference, "tests", "golden", "test_apps")
    if not os.path.isdir(golden):
        if verbose:
            print(f"[oracle/_ref] no reference checkout at {reference}; skipped")
        return None
    objs = []
    units = []
    for stem, fname in (("sgemm", "test_x86_sgemm.txt"), ("conv", "test_x86_conv.txt")):
        header, c_text = _split(os.path.join(golden, fname))
        _write(f"{stem}/test_case.h", header)
        units.append((stem, _write(f"{stem}/{stem}.c", c_text), ["-mavx512f", "-mfma"]))
    units.append(("i8mm", _int8_unit(os.path.join(golden, "test_gemmini_matmul.txt"),
                                     "i8mm", r"^void (cpu_matmul_\w+)\( [^;]*\) \{"), []))
    units.append(("i8conv", _int8_unit(os.path.join(golden, "test_gemmini_conv.txt"),
                                       "i8conv", r"^void (conv_\w+_cpu)\( [^;]*\) \{"), []))
    for stem, src, flags in units:
        obj = os.path.join(OUT, f"{stem}.o")
        cmd = ["gcc", "-O3", "-fPIC", *flags, "-I", os.path.join(OUT, stem), "-c", src, "-o", obj]
        subprocess.run(cmd, check=True)
        objs.append(obj)
    so = os.path.join(OUT, "libexo_ref.so")
    subprocess.run(["gcc", "-shared", "-o", so, *objs, "-lm"], check=True)
    if verbose:
        print(f"[oracle/_ref] built {so}")
    return so


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    args = ap.parse_args()
    sys.exit(0 if build(args.reference) else 1)
