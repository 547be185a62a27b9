"""Pattern discovery oracle (test infrastructure, CPU only).

Restates the SPION-CF pattern step of the reference driver:

    main_conv_ff.py:255-265   diagonal convolution + block average pooling
    main_conv_ff.py:266-268   zero guard row/column and quantile threshold
    main_conv_ff.py:35-62     ``flood_fill``: greedy down/right/diagonal walker
    main_conv_ff.py:271-274   2*nb seeds: first row, then first column
    main_conv_ff.py:276-278   binarise and force the diagonal

and the two sibling variants

    main_conv.py:246-251      SPION-C: top-k of the pooled map instead of walkers
    main_ff.py:255            SPION-F: no convolution (average pool only)

Two flavours of the float stages are provided:

* ``pooled_fixed_order``  - the order of additions is fixed (documented below)
  and carried out in fp64, rounded to fp32 once.  The CUDA kernel uses the
  same order, so both produce identical bits by construction.
* ``pooled_torch``        - the reference's own calls (``F.conv2d`` with
  ``padding='same'`` followed by ``F.avg_pool2d``), whose summation order is
  whatever the CPU backend picks.  Used to pin the fixed-order flavour at the
  level that matters: the resulting block mask.

All integer results (mask, CSR) are compared with ``==`` by the tests.
"""
from __future__ import annotations

import numpy as np

CONV_DIAG = 0   # F x F kernel with ones on the main diagonal (main_conv_ff.py:258-262)
CONV_BOX = 1    # F x F box mean (the "3x3 mean" wording of the benchmark config)


# --------------------------------------------------------------------------- float stages
def conv_fixed_order(A: np.ndarray, F: int = 31, kind: int = CONV_DIAG) -> np.ndarray:
    """'same'-padded convolution of the [L, L] map, fp64, fixed addition order.

    diag:  c[i,j] = sum_{t=-h..h} A[i+t, j+t]            added for t = -h, -h+1, ..., h
    box :  c[i,j] = (sum_{u=-h..h} sum_{v=-h..h} A[i+u, j+v]) / F^2
           added for u outer, v inner, both ascending; one fp64 division at the end.
    Out-of-range taps contribute an explicit +0.0 (zero padding, main_conv_ff.py:263).
    """
    assert F % 2 == 1
    L = A.shape[0]
    h = F // 2
    P = np.zeros((L + 2 * h, L + 2 * h), dtype=np.float64)
    P[h:h + L, h:h + L] = A.astype(np.float64)
    c = np.zeros((L, L), dtype=np.float64)
    if kind == CONV_DIAG:
        for t in range(-h, h + 1):
            c = c + P[h + t:h + t + L, h + t:h + t + L]
    elif kind == CONV_BOX:
        for u in range(-h, h + 1):
            for v in range(-h, h + 1):
                c = c + P[h + u:h + u + L, h + v:h + v + L]
        c = c / np.float64(F * F)
    else:
        raise ValueError("unknown conv kind")
    return c


def pool_fixed_order(c: np.ndarray, bs: int) -> np.ndarray:
    """Block average pooling (main_conv_ff.py:264), fp64, fixed addition order.

    r[i, bj]  = sum_{jj=0..bs-1} c[i, bj*bs + jj]        added for jj ascending
    p[bi, bj] = sum_{ii=0..bs-1} r[bi*bs + ii, bj]       added for ii ascending
    out       = fp32( p / bs^2 )                         one rounding to fp32
    """
    L = c.shape[0]
    nb = L // bs
    c3 = c.reshape(L, nb, bs)
    r = np.zeros((L, nb), dtype=np.float64)
    for jj in range(bs):
        r = r + c3[:, :, jj]
    r3 = r.reshape(nb, bs, nb)
    p = np.zeros((nb, nb), dtype=np.float64)
    for ii in range(bs):
        p = p + r3[:, ii, :]
    return (p / np.float64(bs * bs)).astype(np.float32)


def pooled_fixed_order(A: np.ndarray, bs: int, F: int = 31, kind: int = CONV_DIAG) -> np.ndarray:
    A = np.asarray(A, dtype=np.float32)
    if F == 1:                       # SPION-F: average pool only (main_ff.py:255)
        return pool_fixed_order(A.astype(np.float64), bs)
    return pool_fixed_order(conv_fixed_order(A, F, kind), bs)


def pooled_torch(A, bs: int, F: int = 31, kind: int = CONV_DIAG) -> np.ndarray:
    """The reference's own float stages (main_conv_ff.py:258-265) on CPU tensors."""
    import torch
    import torch.nn.functional as Fnn
    data = torch.as_tensor(np.asarray(A, dtype=np.float32))
    if F > 1:
        if kind == CONV_DIAG:
            kernel = np.zeros((F, F))
            np.fill_diagonal(kernel, 1)
        else:
            kernel = np.full((F, F), 1.0 / (F * F))
        kernel = torch.Tensor(kernel)[None, None]
        out = Fnn.conv2d(data[None], kernel, stride=1, padding='same')
    else:
        out = data[None]
    out = Fnn.avg_pool2d(out, (bs, bs))[0]
    return out.numpy().astype(np.float32)


def _fma32(a, b, c) -> np.float32:
    """fp32 fused multiply-add: a*b is exact in fp64 for fp32 inputs."""
    return np.float32(np.float64(np.float32(a)) * np.float64(np.float32(b)) + np.float64(np.float32(c)))


def quantile_threshold(pooled: np.ndarray, q: float) -> np.float32:
    """``torch.quantile(out, q)`` (main_conv_ff.py:268), linear interpolation.

    Restated from torch's CPU kernel: rank = fp32(q) * fp32(n-1) in fp32; the two
    neighbours are combined with torch's ``lerp``, which is fused:
        w <  0.5 :  fma(w, hi-lo, lo)
        w >= 0.5 :  fma(-(hi-lo), 1-w, hi)
    ``tests/test_oracle_pattern.py`` checks this bit for bit against torch.
    """
    s = np.sort(np.asarray(pooled, dtype=np.float32).ravel(), kind='stable')
    n = s.size
    rank = np.float32(np.float32(q) * np.float32(n - 1))
    lo_i = int(np.floor(rank))
    hi_i = int(np.ceil(rank))
    w = np.float32(rank - np.float32(lo_i))
    lo, hi = s[lo_i], s[hi_i]
    d = np.float32(hi - lo)
    if abs(w) < np.float32(0.5):
        return _fma32(w, d, lo)
    return _fma32(-d, np.float32(np.float32(1.0) - w), hi)


# --------------------------------------------------------------------------- integer stages
def greedy_paths(pooled: np.ndarray, thresh) -> np.ndarray:
    """2*nb walkers of ``flood_fill`` (main_conv_ff.py:35-62, seeds :271-274), iterative.

    Returns the 0/1 uint8 mask *before* the diagonal is forced.
    A destination cell is marked when its value is > thresh; the reference stores the
    value and later tests ``ff_mat > 0`` (:276), so the value must also be > 0.
    """
    pooled = np.asarray(pooled, dtype=np.float32)
    nb = pooled.shape[0]
    g = np.zeros((nb + 1, nb + 1), dtype=np.float32)       # zero guard (:266-267)
    g[:nb, :nb] = pooled
    thresh = np.float32(thresh)
    mat = np.zeros((nb, nb), dtype=np.uint8)
    seeds = [(0, k) for k in range(nb)] + [(k, 0) for k in range(nb)]
    for (x, y) in seeds:
        while not (x + 1 == nb + 1 or y + 1 == nb + 1):     # :37
            D, R, G = g[x + 1, y], g[x, y + 1], g[x + 1, y + 1]
            if D > R:
                if D > G:
                    x, v = x + 1, D
                else:
                    x, y, v = x + 1, y + 1, G
            else:
                if R > G:
                    y, v = y + 1, R
                else:
                    x, y, v = x + 1, y + 1, G
            if v > thresh and v > 0:
                mat[x, y] = 1
    return mat


def force_diagonal(mat: np.ndarray) -> np.ndarray:
    out = mat.copy()
    np.fill_diagonal(out, 1)                                 # main_conv_ff.py:277-278
    return out


def topk_mask(pooled: np.ndarray, density: float) -> np.ndarray:
    """SPION-C (main_conv.py:246-251): k = int(nb^2*density - nb) largest pooled cells.

    ``torch.topk`` on ties returns an implementation-defined subset; the restatement
    (and the CUDA kernel) break ties towards the lower flat index.
    """
    pooled = np.asarray(pooled, dtype=np.float32)
    nb = pooled.shape[0]
    k = int(nb * nb * density - nb)
    mat = np.zeros(nb * nb, dtype=np.uint8)
    if k > 0:
        flat = pooled.ravel()
        order = np.lexsort((np.arange(flat.size), -flat.astype(np.float64)))
        mat[order[:k]] = 1
    return mat.reshape(nb, nb)


def discover_block_mask(A, bs: int, q: float, F: int = 31, kind: int = CONV_DIAG,
                        float_path: str = "fixed"):
    """Full SPION-CF step: returns (mat uint8 [nb,nb], thresh fp32, pooled fp32 [nb,nb])."""
    if float_path == "fixed":
        pooled = pooled_fixed_order(A, bs, F, kind)
    elif float_path == "torch":
        pooled = pooled_torch(A, bs, F, kind)
    else:
        raise ValueError(float_path)
    thresh = quantile_threshold(pooled, q)
    mat = force_diagonal(greedy_paths(pooled, thresh))
    return mat, thresh, pooled


def discover_block_mask_topk(A, bs: int, density: float, F: int = 31, kind: int = CONV_DIAG):
    pooled = pooled_fixed_order(A, bs, F, kind)
    return force_diagonal(topk_mask(pooled, density)), pooled


def stack_for_reference(mats) -> np.ndarray:
    """[4, layers, nb, nb] fp32 form the reference pickles (main_conv_ff.py:298-299)."""
    m = np.stack([np.asarray(x, dtype=np.float32) for x in mats], 0)
    return np.stack([m, m, m, m], 0)
