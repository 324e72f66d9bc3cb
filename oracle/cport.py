"""ctypes binding of oracle/csrc/libbm_oracle.so, the C restatement of the reference's CPU algorithm
(test infrastructure + the timed CPU baseline; see oracle/__init__.py)."""
import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
_LIB = os.path.join(_DIR, "libbm_oracle.so")
_fp = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def _load():
    if not os.path.exists(_LIB):
        subprocess.check_call(["make", "-s", "-C", _DIR])
    lib = C.CDLL(_LIB)
    lib.bm_oracle_max_threads.restype = C.c_int
    lib.bm_oracle_ssd2_serial.restype = C.c_int
    lib.bm_oracle_ssd2_serial.argtypes = [_fp, _fp, _fp, _fp, _fp, _fp, C.c_void_p, _fp, _fp] + [C.c_int] * 8
    lib.bm_oracle_step2.restype = None
    lib.bm_oracle_step2.argtypes = [_fp] * 8 + [C.c_int] * 6
    lib.bm_oracle_selscan1.restype = None
    lib.bm_oracle_selscan1.argtypes = [_fp, _fp, _fp, _fp, _fp, _fp, C.c_void_p, _fp, _fp] + [C.c_int] * 5
    return lib


lib = _load()


def max_threads():
    return lib.bm_oracle_max_threads()


def _h0ptr(h0):
    return None if h0 is None else h0.ctypes.data_as(C.c_void_p)


def ssd2_serial(x, dt, a, b, c, d, h0, chunk_len, nthreads=0):
    bsz, s, h, p = x.shape
    g, r = b.shape[2], b.shape[3]
    y = np.empty_like(x)
    hf = np.empty((bsz, h, p, r), np.float32)
    h0 = None if h0 is None else np.ascontiguousarray(h0, np.float32)
    rc = lib.bm_oracle_ssd2_serial(x, dt, a, b, c, d, _h0ptr(h0), y, hf, bsz, s, h, p, r, g, chunk_len, nthreads)
    if rc != 0:
        raise ValueError("seqlen must be a multiple of chunk_len")
    return y, hf


def step2(state, x, dt, a, b, c, d, nthreads=0):
    bsz, h, p, r = state.shape
    y = np.empty((bsz, h, p), np.float32)
    lib.bm_oracle_step2(state, x, dt, a, b, c, d, y, bsz, h, p, r, b.shape[1], nthreads)
    return y


def selscan1(u, delta, a, b, c, d, h0, nthreads=0):
    bsz, s, di = u.shape
    r = a.shape[1]
    y = np.empty_like(u)
    hf = np.empty((bsz, di, r), np.float32)
    h0 = None if h0 is None else np.ascontiguousarray(h0, np.float32)
    lib.bm_oracle_selscan1(u, delta, a, b, c, d, _h0ptr(h0), y, hf, bsz, s, di, r, nthreads)
    return y, hf
