"""Builds the C oracle (oracle/w8a8_oracle.c) into oracle/_build/libw8a8_oracle.so.

Test infrastructure: only the tests, the smoke check and the benchmark's CPU-baseline
legs load the result.  Run as a script or call build().
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "w8a8_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libw8a8_oracle.so")


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def build(force: bool = False) -> str:
    """Compile if the library is missing or older than its source; returns its path."""
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)
            and os.path.getmtime(OUT) >= os.path.getmtime(__file__)):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    # -O3 vectorises the int8 dot products; floating-point results do not depend on the level
    # (no fast-math, no contraction)
    cmd = ["gcc", "-O3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
           "-std=c11", "-Wall", "-o", OUT, SRC, "-lm"]
    flags = _cpu_flags()
    if "fma" in flags:
        # fmaf() then compiles to one instruction; the value is the same either way
        cmd.insert(1, "-mfma")
    if "avx2" in flags:
        cmd.insert(1, "-mavx2")
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
