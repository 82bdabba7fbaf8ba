"""Makes tests/golden/conv_golden.json from the reference's own host C++.

Only two pieces of zeraix/imparo compile on a machine without its Rust toolchain: the
host functions of imparo-cuda/native/lfm2_ops.cuh (gated short convolution and its state
advance) and kv_paging.cuh.  This script compiles conv_harness.cpp against lfm2_ops.cuh
and records a few cases, among them portions shorter than taps-1 and a non-zero state.

    python tests/golden/make_conv_golden.py /path/to/imparo  (writes conv_golden.json)
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(5, 3, 7, 11), (6, 4, 2, 12), (4, 2, 1, 13), (3, 4, 1, 14), (8, 3, 16, 15), (7, 5, 3, 16)]  # width, taps, tokens, seed


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_conv_golden.py /path/to/imparo (a checkout of zeraix/imparo)")
    ref = sys.argv[1]
    inc = os.path.join(ref, "crates", "imparo-cuda", "native")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "conv_harness")
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", inc, os.path.join(HERE, "conv_harness.cpp"), "-o", exe], check=True)
        cases = [json.loads(subprocess.run([exe] + [str(x) for x in c], check=True, capture_output=True, text=True).stdout)
                 for c in CASES]
    with open(os.path.join(HERE, "conv_golden.json"), "w") as f:
        json.dump({"source": "imparo-cuda/native/lfm2_ops.cuh shortconv_reference + shortconv_state_reference",
                   "cases": cases}, f)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
