"""Writes tests/golden/reference_ffi_symbols.txt: the names in the reference's `extern "C"` FFI block
(src/cuda.rs:87-682). Run where the reference checkout is available: python extract_ffi_symbols.py /path/to/m40-llm"""
import os
import re
import sys

ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
lines = open(os.path.join(ref, "src", "cuda.rs")).read().split("\n")[86:683]
names = sorted(set(re.findall(r"pub fn (m40llm_\w+)", "\n".join(lines))))
open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_ffi_symbols.txt"), "w").write("\n".join(names) + "\n")
print(len(names))
