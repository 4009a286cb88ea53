"""Build recipe for the test oracle (TEST INFRASTRUCTURE, not part of the product).

  python oracle/build.py          builds oracle/_build/libhetu_oracle.so      (1 thread, the checker)
                                   and  oracle/_build/libhetu_oracle_mt.so   (OpenMP, the timed CPU baseline)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
SRC = os.path.join(HERE, "hetu_oracle.cc")


def _stale(target, *sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    jobs = [
        (os.path.join(OUT, "libhetu_oracle.so"), []),
        (os.path.join(OUT, "libhetu_oracle_mt.so"), ["-fopenmp", "-DHO_PARALLEL"]),
    ]
    for target, extra in jobs:
        if not force and not _stale(target, SRC):
            continue
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", *extra, SRC, "-o", target]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return [j[0] for j in jobs]


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
