"""Compiles oracle/void_oracle_c.c (the C restatement of the reference's INT8 SpMM) into oracle/lib/.

Test infrastructure: used by tests/, by __graft_entry__.build() and by bench.py's CPU baseline only.
Run as ``python -m oracle.build_c``.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "void_oracle_c.c")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libvoid_oracle.so")


def build(force: bool = False) -> str:
    """Returns the path of the shared library, or '' when no C compiler is available."""
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(SRC):
        return LIB_PATH
    gcc = shutil.which("gcc")
    if gcc is None:
        return LIB_PATH if os.path.exists(LIB_PATH) else ""
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [gcc, "-O3", "-std=gnu11", "-fopenmp", "-fPIC", "-shared", "-Wall", "-o", LIB_PATH, SRC]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("gcc failed:\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True))
