"""Attention oracle (test infrastructure, CPU only; also the timed CPU baseline).

What the reference's sparse kernels compute (models/block_attn.cu:453-545):

    S   = Q K^T                       only at the selected (block-mask) positions   :459
    v   = S * scale  [ - 1e6*(1-keypad[col]) in the key-padding variant ]           :52, _mask.cu:110
    m   = max(floor, max_sel v)        floor = -100 (:48) or 0 (_mask.cu:105)
    Z   = sum_sel exp(v - m) + (L - n_i) * exp(-m)                                  :65-71
    P   = exp(v - m) / Z               (0 if 1/Z == 0)                              :72-87
    O   = P V                                                                       :478
    dP  = dO V^T at the selected positions                                          :498
    t   = dP * P ;  dS = (t - P * sum_sel t) * scale                                :107-129
    dQ  = dS K ;  dK = dS^T Q ;  dV = P^T dO                                        :516-536

i.e. every non-selected key of a row takes part in the softmax denominator with
score 0 and is then dropped.  In closed form, with M the block mask upsampled to
[L, L]:  P = softmax((S*scale - pad) * M, dim=-1) * M, whose autograd gradient is
exactly the backward above.  ``sparse_attention`` is that closed form;
``sparse_attention_rowwise`` follows the kernel statement by statement and is used
to check the closed form.  The dense warm-up path (models/attn.cu:183-262,
models/attention.py:13-38) is ``dense_attention``.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def expand_mask(mat, bs: int) -> torch.Tensor:
    """Block mask [nb, nb] -> element mask [L, L] (nn.Upsample nearest, attention_blockcuda.py:41)."""
    m = torch.as_tensor(np.asarray(mat)).to(torch.float32)
    return m.repeat_interleave(bs, 0).repeat_interleave(bs, 1)


def sparse_attention(Q, K, V, mat, bs: int, keypad=None, dO=None, dtype=torch.float32):
    """Dense-masked closed form.  Q, K, V: [B, H, L, d].  keypad: [B, L] of 1 (keep) / 0 (pad).

    Returns (O, P_dense) or, when dO is given, (O, P_dense, dQ, dK, dV).
    """
    Q = Q.detach().to(dtype).requires_grad_(dO is not None)
    K = K.detach().to(dtype).requires_grad_(dO is not None)
    V = V.detach().to(dtype).requires_grad_(dO is not None)
    M = expand_mask(mat, bs).to(dtype)
    d = Q.shape[-1]
    S = torch.matmul(Q, K.transpose(-2, -1)) / math.sqrt(d)          # attention.py:28-29
    if keypad is not None:
        S = S - 1e6 * (1 - keypad.to(dtype)[:, None, None, :])       # attention_blockcuda_mask.py:42-43
    P = torch.softmax(S * M, dim=-1) * M
    O = torch.matmul(P, V)
    if dO is None:
        return O.detach(), P.detach()
    O.backward(dO.to(dtype))
    return O.detach(), P.detach(), Q.grad, K.grad, V.grad


def dense_attention(Q, K, V, keypad=None, dO=None, dtype=torch.float32):
    """Plain softmax attention (models/attention.py:13-38 without dropout)."""
    nb = 1
    L = Q.shape[-2]
    return sparse_attention(Q, K, V, np.ones((nb, nb), np.uint8), L, keypad, dO, dtype)


def sparse_attention_rowwise(Q, K, V, mat, bs: int, keypad=None, dO=None, floor=None):
    """Statement-by-statement fp32 emulation of the reference kernels (small shapes only).

    Returns P as a list over (b,h) of per-row value arrays in element-CSR order, plus O and,
    when dO is given, dQ, dK, dV.  Numpy fp32 throughout, like the kernels.
    """
    Q = np.asarray(Q, np.float32); K = np.asarray(K, np.float32); V = np.asarray(V, np.float32)
    B, H, L, d = Q.shape
    scale = np.float32(1.0 / math.sqrt(d))
    if floor is None:
        floor = np.float32(-100.0 if keypad is None else 0.0)
    mat = (np.asarray(mat) != 0)
    cols_of_row = []
    for r in range(L // bs):
        cs = np.nonzero(mat[r])[0]
        cols_of_row.append((cs[:, None] * bs + np.arange(bs)[None, :]).reshape(-1))
    O = np.zeros_like(Q)
    dQ = np.zeros_like(Q); dK = np.zeros_like(Q); dV = np.zeros_like(Q)
    Pvals = []
    for b in range(B):
        for h in range(H):
            rows = []
            for i in range(L):
                cols = cols_of_row[i // bs]
                n_i = cols.size
                v = (K[b, h, cols] @ Q[b, h, i]).astype(np.float32) * scale
                if keypad is not None:
                    v = v - np.float32(1e6) * (np.float32(1) - np.asarray(keypad, np.float32)[b, cols])
                m = max(floor, v.max()) if n_i else floor
                e = np.exp((v - m).astype(np.float32))
                Z = np.float32(e.sum(dtype=np.float32) + np.float32(L - n_i) * np.exp(np.float32(-m)))
                inv = np.float32(1) / Z
                p = np.zeros_like(e) if inv == 0 else (e * inv).astype(np.float32)
                rows.append(p)
                O[b, h, i] = p @ V[b, h, cols]
                if dO is not None:
                    g = np.asarray(dO, np.float32)[b, h, i]
                    dP = V[b, h, cols] @ g
                    t = dP * p
                    dS = (t - p * t.sum(dtype=np.float32)) * scale
                    dQ[b, h, i] = dS @ K[b, h, cols]
                    dK[b, h, cols] += dS[:, None] * Q[b, h, i][None, :]
                    dV[b, h, cols] += p[:, None] * g[None, :]
            Pvals.append(rows)
    if dO is None:
        return Pvals, O
    return Pvals, O, dQ, dK, dV


def sparse_attention_blockwise(Q, K, V, mat, bs: int, keypad=None, dO=None, floor=None):
    """The same semantics block row by block row in numpy fp64, for ONE (b,h) matrix: Q, K, V, dO are
    [L, d]; keypad [L] of 1 (keep) / 0 (pad) or None.  Never forms an [L, L] array, so it reaches the
    largest sequence lengths of the kernel sweep (L = 16384, nb = 512) in seconds.  Follows
    models/block_attn.cu:33-130 per row (maximum with floor, the (L - n) exp(-m) term, backward through
    the selected entries only) and :453-545 for the products.

    Returns (O, P_tiles[, dQ, dK, dV]) with P_tiles [nnzb, bs, bs] in CSR block order.
    """
    Q = np.asarray(Q, np.float64); K = np.asarray(K, np.float64); V = np.asarray(V, np.float64)
    L, d = Q.shape
    nb = L // bs
    scale = 1.0 / math.sqrt(d)
    if floor is None:
        floor = -100.0 if keypad is None else 0.0
    mat = np.asarray(mat) != 0
    g = None if dO is None else np.asarray(dO, np.float64)
    kp = None if keypad is None else np.asarray(keypad, np.float64)
    O = np.zeros((L, d)); dQ = np.zeros((L, d)); dK = np.zeros((L, d)); dV = np.zeros((L, d))
    tiles = []
    for r in range(nb):
        cs = np.nonzero(mat[r])[0]
        rows = slice(r * bs, (r + 1) * bs)
        if cs.size == 0:
            continue
        cols = (cs[:, None] * bs + np.arange(bs)[None, :]).reshape(-1)
        v = (Q[rows] @ K[cols].T) * scale                                  # [bs, n]
        if kp is not None:
            v = v - 1e6 * (1.0 - kp[cols])[None, :]
        m = np.maximum(floor, v.max(axis=1, keepdims=True))
        e = np.exp(v - m)
        Z = e.sum(axis=1, keepdims=True) + (L - cols.size) * np.exp(-m)
        p = e / Z
        tiles.append(p.reshape(bs, cs.size, bs).transpose(1, 0, 2))
        O[rows] = p @ V[cols]
        if g is not None:
            dP = g[rows] @ V[cols].T
            t = dP * p
            dS = (t - p * t.sum(axis=1, keepdims=True)) * scale
            dQ[rows] = dS @ K[cols]
            dK[cols] += dS.T @ Q[rows]
            dV[cols] += p.T @ g[rows]
    P_tiles = np.concatenate(tiles, 0) if tiles else np.zeros((0, bs, bs))
    if g is None:
        return O, P_tiles
    return O, P_tiles, dQ, dK, dV


def csr_values_from_dense(P_dense, mat, bs: int) -> np.ndarray:
    """Gather a dense [B,H,L,L] tensor into the reference's value layout [BH, nnz]
    (element rows in order, selected element columns ascending; attention_blockcuda.py:51,67)."""
    P = np.asarray(P_dense)
    B, H, L, _ = P.shape
    M = expand_mask(mat, bs).numpy().astype(bool)
    return P.reshape(B * H, L, L)[:, M]


def block_values_from_dense(P_dense, mat, bs: int) -> np.ndarray:
    """Gather a dense [B,H,L,L] tensor into block-tile layout [BH, nnzb, bs, bs] (CSR block order)."""
    P = np.asarray(P_dense)
    B, H, L, _ = P.shape
    nb = L // bs
    r, c = np.nonzero(np.asarray(mat) != 0)
    P6 = P.reshape(B * H, nb, bs, nb, bs)
    return np.ascontiguousarray(P6[:, r, :, c, :].transpose(1, 0, 2, 3))


def fwd_bwd_step(Q, K, V, dO, M_elem, keypad=None):
    """One timed CPU-baseline step: dense-masked fwd + autograd bwd, fp32, given a
    pre-expanded element mask (so the expansion is not part of the timed work)."""
    Q = Q.detach().requires_grad_(True); K = K.detach().requires_grad_(True); V = V.detach().requires_grad_(True)
    S = torch.matmul(Q, K.transpose(-2, -1)) / math.sqrt(Q.shape[-1])
    if keypad is not None:
        S = S - 1e6 * (1 - keypad[:, None, None, :])
    P = torch.softmax(S * M_elem, dim=-1) * M_elem
    O = torch.matmul(P, V)
    O.backward(dO)
    return O.detach(), Q.grad, K.grad, V.grad
