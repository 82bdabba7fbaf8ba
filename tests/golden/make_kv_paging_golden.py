"""Makes tests/golden/kv_paging_golden.json from the reference's own page-address rule.

imparo-cuda/native/kv_paging.cuh is plain C++ on the host side and compiles without the
reference's Rust toolchain.  This script compiles kv_paging_harness.cpp against it and records,
for shuffled block tables, the physical cache row of logical positions at page edges and at
scattered places.  The engine's kernels address their pages by the same rule with the page size
as a parameter; the tests compare them at the reference's page size of 64.

    python tests/golden/make_kv_paging_golden.py /path/to/imparo  (writes kv_paging_golden.json)
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(3, 12, 5), (7, 40, 6), (16, 96, 7)]      # blocks in the table, rows asked for, seed


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_kv_paging_golden.py /path/to/imparo (a checkout of zeraix/imparo)")
    inc = os.path.join(sys.argv[1], "crates", "imparo-cuda", "native")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "kv_paging_harness")
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", inc, os.path.join(HERE, "kv_paging_harness.cpp"), "-o", exe], check=True)
        cases = [json.loads(subprocess.run([exe] + [str(x) for x in c], check=True, capture_output=True, text=True).stdout)
                 for c in CASES]
    with open(os.path.join(HERE, "kv_paging_golden.json"), "w") as f:
        json.dump({"source": "imparo-cuda/native/kv_paging.cuh physical_row", "cases": cases}, f)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
