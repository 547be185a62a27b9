"""CSR oracle (test infrastructure, CPU only).

``element_csr`` restates the per-call CSR construction of the reference's sparse
autograd function (models/attention_blockcuda.py:31-43, identical lines in
models/attention_blockcuda_mask.py:26-38) with numpy integer arithmetic:

    sum_mat[L]   int32   number of selected *elements* in each element row
    Offsets[L+1] int32   exclusive prefix sum of sum_mat
    Columns[nnz] int32   ascending element column indices, row after row
                         (the reference repeats this BH times; see ``repeat``)

``block_csr`` / ``block_csc`` give the block-level structures the CUDA kernels use.
"""
from __future__ import annotations

import numpy as np


def element_csr(mat: np.ndarray, bs: int, repeat: int = 1):
    mat = (np.asarray(mat) != 0)
    nb = mat.shape[0]
    L = nb * bs
    per_block_row = mat.sum(axis=1).astype(np.int32) * np.int32(bs)      # :31
    sum_mat = np.repeat(per_block_row, bs).astype(np.int32)              # :32-33
    offsets = np.zeros(L + 1, dtype=np.int32)                            # :35
    offsets[1:] = np.cumsum(sum_mat, dtype=np.int64).astype(np.int32)    # :36-37
    # nearest-neighbour upsample of the block mask, then nonzero()[:, 1]  (:41-42):
    # every element row of block row r lists, for each selected block column c
    # in ascending order, the bs element columns c*bs .. c*bs+bs-1.
    chunks = []
    for r in range(nb):
        cs = np.nonzero(mat[r])[0]
        one_row = (cs[:, None] * bs + np.arange(bs)[None, :]).reshape(-1)
        chunks.append(np.tile(one_row, bs))
    columns = (np.concatenate(chunks) if chunks else np.zeros(0)).astype(np.int32)
    nnz = int(offsets[-1])                                               # :39
    assert columns.size == nnz
    if repeat > 1:
        columns = np.tile(columns, repeat)                               # :43
    return sum_mat, offsets, columns, nnz


def block_csr(mat: np.ndarray):
    """row_ptr[nb+1], col_idx[nnzb] (ascending inside a row), blk_row[nnzb]."""
    mat = (np.asarray(mat) != 0)
    nb = mat.shape[0]
    row_ptr = np.zeros(nb + 1, dtype=np.int32)
    row_ptr[1:] = np.cumsum(mat.sum(axis=1))
    r, c = np.nonzero(mat)
    return row_ptr, c.astype(np.int32), r.astype(np.int32)


def block_csc(mat: np.ndarray):
    """col_ptr[nb+1], row_idx[nnzb] (ascending inside a column), csr_pos[nnzb].

    csr_pos[p] is the position (block id) of CSC entry p inside the CSR ordering.
    """
    mat = (np.asarray(mat) != 0)
    nb = mat.shape[0]
    csr_id = np.full((nb, nb), -1, dtype=np.int64)
    r, c = np.nonzero(mat)
    csr_id[r, c] = np.arange(r.size)
    col_ptr = np.zeros(nb + 1, dtype=np.int32)
    col_ptr[1:] = np.cumsum(mat.sum(axis=0))
    cc, rr = np.nonzero(mat.T)
    return col_ptr, rr.astype(np.int32), csr_id[rr, cc].astype(np.int32)
