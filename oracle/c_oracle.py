"""ctypes binding of the plain-C restatement (oracle/spion_oracle.c); test infrastructure only.

``load()`` builds the library on first use when a C compiler is present and returns None otherwise, so callers
(the tests, the CPU-baseline leg of bench.py) can fall back to the numpy / torch restatement.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_LIB = None
_F = ctypes.POINTER(ctypes.c_float)
_U8 = ctypes.POINTER(ctypes.c_uint8)
_I32 = ctypes.POINTER(ctypes.c_int32)


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    from . import build_c
    try:
        path = build_c.build()
    except (RuntimeError, OSError):
        if not os.path.exists(build_c.OUT):
            return None
        path = build_c.OUT
    lib = ctypes.CDLL(path)
    lib.oracle_threads.restype = ctypes.c_int
    lib.oracle_discover.argtypes = [_F, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_double, _U8, _F, _F]
    lib.oracle_block_csr.argtypes = [_U8, ctypes.c_int] + [_I32] * 6
    lib.oracle_element_csr.argtypes = [_U8, ctypes.c_int, ctypes.c_int, ctypes.c_int, _I32, _I32, _I32]
    lib.oracle_element_csr.restype = ctypes.c_longlong
    lib.oracle_attention_step.argtypes = [_F, _F, _F, _F, _F, ctypes.c_float, _U8] + [ctypes.c_int] * 4 + [_F] * 6
    _LIB = lib
    return lib


def _f(a):
    return a.ctypes.data_as(_F) if a is not None else None


def discover(A, bs: int, param: float, F: int = 31, kind: int = 0, select: str = "quantile"):
    """(mat uint8 [nb,nb], thresh fp32, pooled fp32 [nb,nb]) like oracle.pattern.discover_block_mask[_topk]."""
    lib = load()
    A = np.ascontiguousarray(A, dtype=np.float32)
    L = A.shape[0]
    nb = L // bs
    mat = np.zeros((nb, nb), np.uint8)
    pooled = np.zeros((nb, nb), np.float32)
    thresh = ctypes.c_float(0)
    rc = lib.oracle_discover(_f(A), L, bs, F, kind, 0 if select == "quantile" else 1, float(param),
                             mat.ctypes.data_as(_U8), _f(pooled), ctypes.byref(thresh))
    if rc:
        raise RuntimeError(f"oracle_discover failed ({rc})")
    return mat, np.float32(thresh.value), pooled


def block_csr(mat):
    lib = load()
    mat = np.ascontiguousarray(np.asarray(mat) != 0, dtype=np.uint8)
    nb = mat.shape[0]
    arrs = [np.zeros(nb + 1, np.int32), np.zeros(nb * nb, np.int32), np.zeros(nb * nb, np.int32),
            np.zeros(nb + 1, np.int32), np.zeros(nb * nb, np.int32), np.zeros(nb * nb, np.int32)]
    n = lib.oracle_block_csr(mat.ctypes.data_as(_U8), nb, *[a.ctypes.data_as(_I32) for a in arrs])
    row_ptr, col_idx, blk_row, col_ptr, row_idx, csc_pos = arrs
    return row_ptr, col_idx[:n], blk_row[:n], col_ptr, row_idx[:n], csc_pos[:n]


def element_csr(mat, bs: int, repeat: int = 1):
    lib = load()
    mat = np.ascontiguousarray(np.asarray(mat) != 0, dtype=np.uint8)
    nb = mat.shape[0]
    L = nb * bs
    nnz_max = int(mat.sum()) * bs * bs
    sum_mat = np.zeros(L, np.int32); offsets = np.zeros(L + 1, np.int32)
    columns = np.zeros(max(1, nnz_max * repeat), np.int32)
    nnz = lib.oracle_element_csr(mat.ctypes.data_as(_U8), nb, bs, repeat, sum_mat.ctypes.data_as(_I32),
                                 offsets.ctypes.data_as(_I32), columns.ctypes.data_as(_I32))
    return sum_mat, offsets, columns[:nnz * repeat], int(nnz)


def attention_step(Q, K, V, mat, bs: int, dO=None, penalty=None, floor=None):
    """Q, K, V, dO: [B, H, L, d] fp32 arrays.  penalty: [B*H, L] (1e6 on padded keys) or None.
    Returns (O, P[BH, nnz]) or (O, P, dQ, dK, dV)."""
    lib = load()
    Q, K, V = [np.ascontiguousarray(x, dtype=np.float32) for x in (Q, K, V)]
    B, H, L, d = Q.shape
    mat = np.ascontiguousarray(np.asarray(mat) != 0, dtype=np.uint8)
    nnz = int(mat.sum()) * bs * bs
    O = np.empty_like(Q); P = np.empty((B * H, nnz), np.float32)
    back = dO is not None
    dOc = np.ascontiguousarray(dO, dtype=np.float32) if back else None
    dS = np.empty((B * H, nnz), np.float32) if back else None
    dQ, dK, dV = (np.empty_like(Q), np.empty_like(Q), np.empty_like(Q)) if back else (None, None, None)
    pen = np.ascontiguousarray(penalty, dtype=np.float32) if penalty is not None else None
    if floor is None:
        floor = -100.0 if pen is None else 0.0
    rc = lib.oracle_attention_step(_f(Q), _f(K), _f(V), _f(dOc), _f(pen), ctypes.c_float(floor),
                                   mat.ctypes.data_as(_U8), B * H, L, d, bs, _f(O), _f(P), _f(dS), _f(dQ), _f(dK),
                                   _f(dV))
    if rc:
        raise RuntimeError(f"oracle_attention_step failed ({rc})")
    return (O, P, dQ, dK, dV) if back else (O, P)
