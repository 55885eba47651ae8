"""Writes tests/golden/generated_prototypes.txt: the public prototypes that exocc
wrote into the generated headers of the three apps on the hot path, one per
line, exactly as they stand in the reference's golden files
(tests/golden/test_apps/test_{x86_sgemm,x86_conv,gemmini_matmul,gemmini_conv}.txt).
tests/test_abi.py compares include/exo_b200.h with them line for line.

    python tests/golden/make_prototypes.py [reference checkout]
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ["test_x86_sgemm.txt", "test_x86_conv.txt", "test_gemmini_matmul.txt", "test_gemmini_conv.txt"]


def main():
    # the exo-lang/exo checkout: argument, else $EXO_REFERENCE, else a "reference" directory beside this repository
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "EXO_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
    out = []
    for f in FILES:
        text = open(os.path.join(ref, "tests", "golden", "test_apps", f)).read()
        header = text.split('#include "test_case.h"')[0]  # the .h part comes first
        for line in header.splitlines():
            if re.match(r"^void \w+\(.*\);\s*$", line):
                out.append(f"{f}: {line.strip()}")
    with open(os.path.join(HERE, "generated_prototypes.txt"), "w") as fh:
        fh.write("\n".join(out) + "\n")
    print(f"{len(out)} prototypes")


if __name__ == "__main__":
    main()
