"""Builds tests/golden/ref_driver.cpp against the reference's own src/qwen_ops.cpp and src/sampler.cpp
(compiled unmodified with g++, on the CPU) and stores what they compute in tests/golden/ref_ops.json.

    python tests/golden/make_golden.py /path/to/reference

The reference's model forward (src/qwen_model.cpp) cannot be built without the HIP runtime, so the golden
values cover the operators and the sampler; tests/test_plain.py compares the plain implementation with
them.  ``hip/hip_fp16.h`` is stood in for by a float-backed ``__half``, which makes the reference's fp16
cache exact; the test feeds values that are exactly representable either way.
"""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
SHIM = """#pragma once
struct __half { float v; };
static inline float __half2float(__half h) { return h.v; }
static inline __half __float2half(float f) { __half h; h.v = f; return h; }
"""


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "hip"))
        with open(os.path.join(tmp, "hip", "hip_fp16.h"), "w") as f:
            f.write(SHIM)
        exe = os.path.join(tmp, "ref_driver")
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", tmp, "-I", os.path.join(ref, "src"),
                               os.path.join(HERE, "ref_driver.cpp"), os.path.join(ref, "src", "qwen_ops.cpp"),
                               os.path.join(ref, "src", "sampler.cpp"), "-o", exe])
        out = subprocess.check_output([exe], text=True)
    with open(os.path.join(HERE, "ref_ops.json"), "w") as f:
        f.write(out)
    print("wrote", os.path.join(HERE, "ref_ops.json"), len(out), "bytes")


if __name__ == "__main__":
    main()
