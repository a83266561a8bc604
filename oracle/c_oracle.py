"""ctypes loader for the C restatement of the oracle (oracle/bqq_oracle.c).

TEST INFRASTRUCTURE ONLY: used by the test-suite and by the CPU-baseline /
reference arm of bench.py; never by the product path."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, 'libbqq_oracle.so')


def load():
    if not os.path.exists(_LIB):
        subprocess.run(['make', '-C', _HERE, '-s'], check=True)
    lib = C.CDLL(_LIB)
    lib.bqq_oracle_forward.restype = C.c_int
    lib.bqq_oracle_forward.argtypes = [C.c_void_p] * 8 + [C.c_int] * 7 + [C.c_void_p, C.c_int, C.c_int]
    lib.bqq_oracle_max_threads.restype = C.c_int
    return lib


def forward(Y, Z, a, b, c, d, X, bias=None, use_double=False, nthreads=0):
    """Y bool [bw,rw,cw,P,r], Z bool [bw,rw,cw,r,Q], a/b/c [bw,rw,cw,1,1], d [rw,cw,1,1], X [M,in]."""
    lib = load()
    Yu = np.ascontiguousarray(np.asarray(Y).astype(np.uint8))
    Zu = np.ascontiguousarray(np.asarray(Z).astype(np.uint8))
    bw, rw, cw, P, r = Yu.shape
    Q = Zu.shape[-1]
    f = lambda t: np.ascontiguousarray(np.asarray(t, np.float32).reshape(-1))
    a_, b_, c_, d_ = f(a), f(b), f(c), f(d)
    X2 = np.ascontiguousarray(np.asarray(X, np.float32).reshape(-1, cw * Q))
    M = X2.shape[0]
    y = np.empty((M, rw * P), np.float32)
    bias_ = f(bias) if bias is not None else None
    rc = lib.bqq_oracle_forward(Yu.ctypes.data, Zu.ctypes.data, a_.ctypes.data, b_.ctypes.data, c_.ctypes.data,
                                d_.ctypes.data, bias_.ctypes.data if bias_ is not None else None, X2.ctypes.data,
                                M, bw, rw, cw, P, Q, r, y.ctypes.data, int(use_double), int(nthreads))
    if rc != 0:
        raise MemoryError('bqq_oracle_forward failed')
    return y


def max_threads():
    return load().bqq_oracle_max_threads()
