"""Compiles oracle/plq_oracle.c into oracle/libplq_oracle.so with gcc (OpenMP).

The reference itself is pure Python on this path, so there is no `oracle/_ref` binary to build:
the C file is a port ("kind": "port" in the benchmark's cpu_baseline)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "plq_oracle.c")
LIB = os.path.join(HERE, "libplq_oracle.so")


def build_oracle(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("gcc failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build_oracle(force=True))
