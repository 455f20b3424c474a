"""geistlib_b200 — B200 (sm_100a) token-sampling path behind geistlib's sampler API.

The product is ``libgeist_b200.so`` (C ABI, declared in ``include/geist_b200.h``).
This package is the thin ctypes view of it that the tests and ``bench.py`` use;
it holds no numeric code and has no fallback: importing :mod:`geistlib_b200.api`
raises if the shared library is missing.
"""
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libgeist_b200.so"
if os.environ.get("GEIST_B200_LIB"):  # an alternative build of the same library (instrumented, debug)
    LIB_PATH = Path(os.environ["GEIST_B200_LIB"])
HEADER_PATH = PKG_DIR.parent / "include" / "geist_b200.h"


def build(verbose: bool = False) -> Path:
    """Compile libgeist_b200.so for sm_100a with nvcc (no GPU needed)."""
    import subprocess

    subprocess.run(["make", "-C", str(PKG_DIR / "csrc")], check=True,
                   stdout=None if verbose else subprocess.DEVNULL)
    return LIB_PATH
