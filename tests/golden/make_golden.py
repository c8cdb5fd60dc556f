"""Regenerates tests/golden/golden.npz by compiling gen_golden.cpp against the
reference tree's headers and running it.  Needs the reference checkout
(a `reference` directory beside this repository, or $Q4T_REFERENCE); the committed golden.npz is what
the tests read, so this only has to run where the reference is available.

    python tests/golden/make_golden.py
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("Q4T_REFERENCE", os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference")))


def main() -> int:
    if not os.path.exists(os.path.join(REF, "include/q4t/quant/format.h")):
        print("reference tree not found at", REF)
        return 1
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "gen_golden")
        subprocess.run(["g++", "-O2", "-std=c++20", "-ffp-contract=off", f"-I{REF}/include",
                        os.path.join(HERE, "gen_golden.cpp"), "-o", exe], check=True)
        manifest = subprocess.run([exe, tmp], check=True, capture_output=True, text=True).stdout
        arrays = {}
        for line in manifest.strip().splitlines():
            name, dtype, *shape = line.split()
            arrays[name] = np.fromfile(os.path.join(tmp, name + ".bin"), dtype="<" + dtype).reshape(
                [int(s) for s in shape])
        np.savez_compressed(os.path.join(HERE, "golden.npz"), **arrays)
        print("wrote golden.npz:", {k: v.shape for k, v in arrays.items()})
    return 0


if __name__ == "__main__":
    sys.exit(main())
