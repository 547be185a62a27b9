"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

They stand in for the LRA image / text / retrieval records (which are not shipped
with the reference: its ``data/`` folder is git-ignored).  Everything is generated
with the CPU torch generator so that a seed means the same tensors on every machine.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def qkv(seed: int, B: int, H: int, L: int, d: int, n: int = 4, dtype=torch.float32):
    """n tensors ~ N(0,1) of shape [B, H, L, d] (Q, K, V, dO for n = 4)."""
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(B, H, L, d, generator=g, dtype=torch.float32).to(dtype) for _ in range(n))


def mean_attention_map(Q: torch.Tensor, K: torch.Tensor) -> torch.Tensor:
    """A = mean over batch, then heads, of softmax(Q K^T / sqrt(d)): the [L, L] map the
    reference's encoder hands to pattern discovery (models/model_transformer.py:137)."""
    d = Q.shape[-1]
    S = torch.matmul(Q.float(), K.float().transpose(-2, -1)) / math.sqrt(d)
    return torch.softmax(S, dim=-1).mean(dim=0).mean(dim=0).contiguous()


def structured_map(seed: int, L: int, n_diag: int = 3, n_vert: int = 4) -> torch.Tensor:
    """Row-stochastic [L, L] map with off-diagonal bands and vertical stripes over noise,
    the shapes trained attention maps show (the reference's figs/patternall.png)."""
    g = torch.Generator().manual_seed(seed)
    S = torch.randn(L, L, generator=g) * 0.5
    i = torch.arange(L)[:, None]
    j = torch.arange(L)[None, :]
    S = S + 4.0 * torch.exp(-((i - j).float() / 6.0) ** 2)
    offs = torch.randint(-L // 2, L // 2, (n_diag,), generator=g)
    for o in offs.tolist():
        S = S + 3.0 * torch.exp(-(((i - j) - o).float() / 4.0) ** 2)
    cols = torch.randint(0, L, (n_vert,), generator=g)
    for c in cols.tolist():
        S = S + 2.5 * torch.exp(-((j - c).float() / 3.0) ** 2)
    return torch.softmax(S, dim=-1).contiguous()


def band_random_mask(seed: int, nb: int, density: float, band: int = 2) -> np.ndarray:
    """Kernel-sweep mask: a diagonal band ``band`` blocks wide (block columns r-band+1 .. r of
    block row r) plus uniformly random off-band blocks up to ``density`` of all nb^2 blocks."""
    rng = np.random.default_rng(seed)
    mat = np.zeros((nb, nb), dtype=np.uint8)
    for r in range(nb):
        mat[r, max(0, r - band + 1):r + 1] = 1
    want = int(round(density * nb * nb))
    extra = want - int(mat.sum())
    if extra > 0:
        free = np.flatnonzero(mat.ravel() == 0)
        pick = rng.choice(free, size=min(extra, free.size), replace=False)
        mat.ravel()[pick] = 1
    return mat


def token_ids(seed: int, B: int, L: int, vocab: int = 256) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (B, L), generator=g)


def labels(seed: int, B: int, n_classes: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 7919)
    return torch.randint(0, n_classes, (B,), generator=g)


def key_padding(seed: int, B: int, L: int, min_keep: float = 0.5) -> torch.Tensor:
    """[B, L] float mask of 1 (token) / 0 (padding tail), as dataset_LRA.py:34 builds from ids != 0."""
    g = torch.Generator().manual_seed(seed + 104729)
    keep = (torch.rand(B, generator=g) * (1 - min_keep) + min_keep) * L
    return (torch.arange(L)[None, :] < keep.long()[:, None]).float()
