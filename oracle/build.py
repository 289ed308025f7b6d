"""Builds the CPU oracle (test infrastructure) into oracle/libfjo_oracle.so with gcc.

No fast-math and no FMA contraction: the restatement must add and multiply in the same order
and with the same roundings as the reference's scalar Rust code.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["fjo_ops.cpp", "fjo_program.cpp", "fjo_paged.cpp", "fjo_pool.cpp", "fjo_sched.cpp"]
HEADERS = ["fjo.h", "fjo_convert.h"]
OUTPUT = os.path.join(HERE, "libfjo_oracle.so")


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    built = os.path.getmtime(OUTPUT)
    return any(os.path.getmtime(os.path.join(HERE, f)) > built for f in SOURCES + HEADERS)


def build(force: bool = False) -> str:
    if not force and not needs_build():
        return OUTPUT
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-fno-fast-math", "-Wall", "-Wextra", "-Wno-unused-parameter", "-o", OUTPUT]
    cmd += [os.path.join(HERE, s) for s in SOURCES]
    subprocess.check_call(cmd, cwd=HERE)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
