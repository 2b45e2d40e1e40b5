"""Build recipe for the CPU oracle (test infrastructure, not the product).

Compiles ``oracle/vkop_oracle.c`` into ``oracle/libvkop_oracle.so`` with gcc.
The reference's own implementation of this path is GLSL compute shaders plus
C++ translation units that include the Vulkan wrapper, so there is nothing of
it that compiles here as plain C/C++; ``oracle/_ref`` is therefore not built.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "vkop_oracle.c")
LIB = os.path.join(HERE, "libvkop_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-Wall", "-Wextra",
           "-o", LIB + ".tmp", SRC, "-lm"]
    subprocess.run(cmd, check=True)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
