"""Compile the C part of the oracle into oracle/_build/liboracle.so and bind it.
TEST INFRASTRUCTURE -- not a product code path."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "liboracle.so")


def build(force=False) -> str:
    src = os.path.join(HERE, "wkv7_seq.c")
    if force or not os.path.exists(OUT) or os.path.getmtime(OUT) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(OUT), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
                        "-o", OUT, src], check=True)
    return OUT


def wkv7_seq(r, w, k, v, a, b, h_in):
    """numpy front end of wkv7_seq.c; returns (out, h_out)."""
    lib = C.CDLL(build())
    B, T, H, S = r.shape
    f = lambda x: np.ascontiguousarray(x, dtype=np.float32)
    arrs = [f(x) for x in (r, w, k, v, a, b, h_in)]
    out = np.empty((B, T, H, S), np.float32)
    h_out = np.empty((B, H, S, S), np.float32)
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    lib.wkv7_seq.argtypes = [C.c_void_p] * 9 + [C.c_int] * 4
    lib.wkv7_seq(*[p(x) for x in arrs], p(out), p(h_out), B, T, H, S)
    return out, h_out
