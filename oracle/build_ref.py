"""Builds ``oracle/_ref``: the reference's OWN CPU statements of this path, compiled from its sources.

TEST INFRASTRUCTURE ONLY.  Nothing of the reference is copied into the repository: at build time the
four function bodies below are cut out of the reference checkout (located by their signatures, ended
by brace matching), written to ``oracle/_ref/*.inc`` (git-ignored) and compiled into two shared
objects together with the shims of this directory (``ref_shim.cpp``, ``ref_shim_nms.cpp``), which
only supply what the bodies need around them (a class to be a member of, C entry points).

  core/function.cpp     Function::get_top_k_predictions   softmax + std::sort top-k of one row
  tests/SoftmaxTest.cpp softmax_nd                        softmax along one axis of an NCHW tensor
  tests/TopkTest.cpp    get_top_k_predictions             std::sort top-k of every row
  tests/NmsTest.cpp     NmsTest::compute_expected_nms     greedy NMS per (batch, class), on libtorch

The reference checkout is looked for at ``$VKOP_REFERENCE`` (default: the read-only mount of the build
container).  Where it is absent (a GPU box), ``build()`` does nothing and whatever ``oracle/_ref``
already holds is used as it is.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("VKOP_REFERENCE", "/root/reference")
LIB = os.path.join(OUT, "libvkop_ref.so")
LIB_NMS = os.path.join(OUT, "libvkop_ref_nms.so")

# (reference file, text inside the declaration, name of the extract, the return type sits on the line before)
EXTRACTS = [
    ("core/function.cpp", "Function::get_top_k_predictions(", "function_get_top_k_predictions.inc", True),
    ("tests/SoftmaxTest.cpp", "void softmax_nd(", "softmax_nd.inc", False),
    ("tests/TopkTest.cpp", "get_top_k_predictions(const std::vector<std::vector<float>>", "topk_get_top_k_predictions.inc", False),
    ("tests/NmsTest.cpp", "compute_expected_nms(const torch::Tensor", "nms_compute_expected_nms.inc", False),
]


def reference_present() -> bool:
    return all(os.path.exists(os.path.join(REFERENCE, f)) for f, _, _, _ in EXTRACTS)


def _cut_function(text: str, marker: str, type_on_line_before: bool) -> tuple[str, int, int]:
    """The definition whose declaration contains `marker`: from the start of the marker's line (or of the line
    before it) to the matching closing brace.  Returns (source, first line, last line), lines counted from 1."""
    at = text.index(marker)
    start = text.rfind("\n", 0, at) + 1
    if type_on_line_before:
        start = text.rfind("\n", 0, start - 1) + 1
    depth, i = 0, text.index("{", at)
    while True:
        c = text[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                break
        i += 1
    return text[start:i + 1] + "\n", text.count("\n", 0, start) + 1, text.count("\n", 0, i) + 1


def extract() -> dict:
    """Writes the extracts; returns {extract name: "file:first-last"}."""
    os.makedirs(OUT, exist_ok=True)
    where = {}
    for rel, marker, name, before in EXTRACTS:
        with open(os.path.join(REFERENCE, rel), encoding="utf-8") as f:
            src, a, b = _cut_function(f.read(), marker, before)
        with open(os.path.join(OUT, name), "w", encoding="utf-8") as f:
            f.write(src)
        where[name] = f"{rel}:{a}-{b}"
    with open(os.path.join(OUT, "EXTRACTED_FROM.txt"), "w") as f:
        for name, loc in where.items():
            f.write(f"{name}\t{loc}\n")
    return where


def _stale(target: str, deps) -> bool:
    return not os.path.exists(target) or any(os.path.getmtime(d) > os.path.getmtime(target) for d in deps)


def build(force: bool = False, with_nms: bool = True) -> str | None:
    """Extracts and compiles; returns the path of libvkop_ref.so, or None when there is neither a reference
    checkout nor a library built earlier."""
    if not reference_present():
        return LIB if os.path.exists(LIB) else None
    shim, shim_nms = os.path.join(HERE, "ref_shim.cpp"), os.path.join(HERE, "ref_shim_nms.cpp")
    srcs = [os.path.join(REFERENCE, f) for f, _, _, _ in EXTRACTS]
    if force or _stale(LIB, srcs + [shim, __file__]):
        extract()
        # plain IEEE arithmetic: no contraction, no fast-math, as the reference's own build (-O0) gives
        cmd = ["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-I", HERE, shim,
               "-o", LIB + ".tmp"]
        subprocess.run(cmd, check=True)
        os.replace(LIB + ".tmp", LIB)
    if with_nms and (force or _stale(LIB_NMS, srcs + [shim_nms, __file__])):
        extract()
        import torch  # the reference's NMS expectation is written on libtorch; the torch wheel ships it

        tdir = os.path.dirname(torch.__file__)
        inc = [os.path.join(tdir, "include"), os.path.join(tdir, "include", "torch", "csrc", "api", "include")]
        cmd = ["g++", "-std=c++17", "-O1", "-ffp-contract=off", "-shared", "-fPIC", "-w",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}", "-I", HERE]
        for i in inc:
            cmd += ["-isystem", i]
        cmd += [shim_nms, "-o", LIB_NMS + ".tmp", "-L", os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-lc10",
                f"-Wl,-rpath,{os.path.join(tdir, 'lib')}"]
        subprocess.run(cmd, check=True)
        os.replace(LIB_NMS + ".tmp", LIB_NMS)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
    with open(os.path.join(OUT, "EXTRACTED_FROM.txt")) as f:
        print(f.read())
