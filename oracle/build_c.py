"""Compile the C restatement of the oracle (oracle/tbik_ref.c) into oracle/libtbik_oracle.so with gcc.

Test infrastructure: called by the build entry point and, on demand, by oracle/c_oracle.py.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "tbik_ref.c")
LIB = os.path.join(HERE, "libtbik_oracle.so")


def build(force: bool = False) -> str:
    if force or not os.path.isfile(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-Wall", "-o", LIB, SRC], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
