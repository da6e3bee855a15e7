"""Compile, from the reference tree itself, the pieces of the hot path that are plain C++ --
so that the CPU checker (attn_oracle.cpp) can be pinned to reference code bit for bit.

    python oracle/build_ref.py [--reference /path/to/llm_simple]     ->  oracle/_ref/libref_pins.so

What is built, always from the files where they lie in the reference tree (nothing of them is
copied into this repository; oracle/_ref/ is not under version control):

  compiled unmodified, with stand-in headers for the third-party includes (oracle/ref_stubs/):
    src/util.cpp                   -> fp32_to_bfloat16                       (src/util.cpp:33-72)
    tests/npu_op_test_util.cpp     -> all_close, InitFreqCIS (test twin)     (:33-48, :109-142)
  extracted at build time into oracle/_ref/*.inc (the enclosing files need Eigen / the Ascend
  runtime and cannot be compiled whole) and compiled inside oracle/ref_wrap.cpp:
    src/model_base.cpp             -> ModelBase::InitFreqCIS                 (:27-83)
    tests/rope_single_layer_test.cpp -> the golden loop of RoPESingleOpTest::Run   (:78-95)
    tests/flash_attn_test.cpp      -> the mask loop of FlashAttentionOpTest::Run   (:124-132)

The two contractions of the attention golden (Eigen tensor contractions) cannot be built without
Eigen; they stay restated in the checker.  Compiled like the reference builds (its CMake files set
only -std=c++20), plus -O2 and -ffp-contract=off: on this x86-64 baseline no fused multiply-add
exists to contract to, the flag only says so.  Test infrastructure: nothing shipped loads the result.
"""
import argparse
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libref_pins.so")
DEFAULT_REFERENCE = os.environ.get("LLM_SIMPLE_REFERENCE", "/root/reference")
CXXFLAGS = ["-std=c++20", "-O2", "-fPIC", "-ffp-contract=off", "-fopenmp"]


def _block_from(text, start_pattern, what):
    """The statement that starts at the first match of start_pattern and runs to its closing brace."""
    m = re.search(start_pattern, text)
    if not m:
        raise RuntimeError("cannot find %s in the reference" % what)
    i = text.index("{", m.start())
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[m.start():j + 1]
    raise RuntimeError("unbalanced braces after %s" % what)


def extract(reference):
    def read(rel):
        with open(os.path.join(reference, rel), encoding="utf-8") as f:
            return f.read()
    pieces = {
        # the whole member function, signature included
        "init_freq_cis.inc": _block_from(read("src/model_base.cpp"),
                                         r"bool\s+ModelBase::InitFreqCIS\s*\(", "ModelBase::InitFreqCIS"),
        # the triple loop over (s, n, f) that fills golden_fp32
        "rope_golden_loop.inc": _block_from(read("tests/rope_single_layer_test.cpp"),
                                            r"for\s*\(\s*int\s+s\s*=\s*0\s*;\s*s\s*<\s*seq_len", "the RoPE golden loop"),
        # the double loop over (row, col) that fills host_mask
        "mask_loop.inc": _block_from(read("tests/flash_attn_test.cpp"),
                                     r"for\s*\(\s*int\s+row\s*=\s*0\s*;\s*row\s*<\s*m", "the mask loop"),
    }
    for name, body in pieces.items():
        with open(os.path.join(OUT, name), "w", encoding="utf-8") as f:
            f.write(body + "\n")


def build(reference=DEFAULT_REFERENCE, force=False):
    """Returns the library path, or None when the reference tree is not present (then a library
    built earlier, if any, is used as it is)."""
    if not os.path.isdir(os.path.join(reference, "src")):
        return LIB if os.path.exists(LIB) else None
    os.makedirs(OUT, exist_ok=True)
    srcs = [os.path.join(reference, "src/util.cpp"), os.path.join(reference, "tests/npu_op_test_util.cpp"),
            os.path.join(reference, "src/model_base.cpp"), os.path.join(reference, "tests/rope_single_layer_test.cpp"),
            os.path.join(reference, "tests/flash_attn_test.cpp"), os.path.join(HERE, "ref_wrap.cpp"), __file__]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(s) <= os.path.getmtime(LIB) for s in srcs):
        return LIB
    extract(reference)
    inc = ["-I", os.path.join(HERE, "ref_stubs"), "-I", os.path.join(reference, "src"),
           "-I", os.path.join(reference, "tests"), "-I", os.path.join(reference, "prebuild")]
    objs = []
    for src, obj in ((srcs[0], "util.o"), (srcs[1], "npu_op_test_util.o"), (srcs[5], "ref_wrap.o")):
        o = os.path.join(OUT, obj)
        subprocess.check_call(["g++"] + CXXFLAGS + inc + ["-I", OUT, "-c", src, "-o", o])
        objs.append(o)
    subprocess.check_call(["g++", "-shared", "-fopenmp", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    path = build(a.reference, a.force)
    print(path if path else "reference tree not found at %s: nothing built" % a.reference)
    sys.exit(0)
