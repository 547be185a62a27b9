"""Pin the pattern / CSR oracle against outputs of the reference's own Python
(fixtures in tests/golden made by tests/golden/make_golden.py)."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import csr as ocsr
from oracle import pattern as opat
from spion_b200 import synthetic

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest()


def _load(name):
    z = np.load(os.path.join(GOLD, name))
    cases = sorted({k.split("/")[0] for k in z.files})
    return z, cases


PAT, PAT_CASES = _load("pattern_reference.npz")


def _map(meta):
    seed, L, bs, F, ck, mk = [int(x) for x in meta]
    if mk == 0:
        Q, K = synthetic.qkv(seed, 2, 2, L, 32, n=2)
        A = synthetic.mean_attention_map(Q, K)
    else:
        A = synthetic.structured_map(seed, L)
    return A.numpy(), L, bs, F, ck


@pytest.mark.parametrize("case", PAT_CASES)
def test_mask_matches_reference(case):
    A, L, bs, F, ck = _map(PAT[case + "/meta"])
    assert _sha(A) == PAT[case + "/sha"].tobytes(), "seeded input differs from the one the fixture was made from"
    nb = L // bs
    gold = np.unpackbits(PAT[case + "/mat"])[:nb * nb].reshape(nb, nb)
    q = float(PAT[case + "/q"])
    # the reference's own float stages + restated walkers: must be identical
    mat_t, thr_t, pooled_t = opat.discover_block_mask(A, bs, q, F, ck, float_path="torch")
    assert np.array_equal(pooled_t, PAT[case + "/pooled"])
    assert np.float32(thr_t) == np.float32(PAT[case + "/thresh"])
    assert np.array_equal(mat_t, gold)
    # fixed-order fp64 float stages (what the CUDA kernel computes): same mask
    mat_f, thr_f, pooled_f = opat.discover_block_mask(A, bs, q, F, ck, float_path="fixed")
    np.testing.assert_allclose(pooled_f, pooled_t, rtol=2e-5, atol=1e-9)
    assert np.array_equal(mat_f, gold)
    # CSR of that mask, restated, hashes to what the reference's torch lines produced
    sm, off, col, nnz = ocsr.element_csr(gold, bs, 1)
    assert nnz == int(PAT[case + "/nnz"])
    assert _sha(np.concatenate([sm, off, col])) == PAT[case + "/csr_sha"].tobytes()


def test_csr_vectors_in_full():
    z, cases = _load("csr_reference.npz")
    for c in cases:
        mat, bs = z[c + "/mat"], int(z[c + "/bs"])
        sm, off, col, nnz = ocsr.element_csr(mat, bs, 2)
        assert nnz == int(z[c + "/nnz"])
        assert np.array_equal(sm, z[c + "/sum_mat"]) and sm.dtype == np.int32
        assert np.array_equal(off, z[c + "/offsets"]) and off.dtype == np.int32
        assert np.array_equal(col, z[c + "/columns"]) and col.dtype == np.int32


def test_block_csr_csc_consistent():
    for seed in range(5):
        mat = synthetic.band_random_mask(seed, 12, 0.3)
        rp, ci, br = ocsr.block_csr(mat)
        cp, ri, pos = ocsr.block_csc(mat)
        assert rp[-1] == cp[-1] == mat.sum()
        for p in range(len(ri)):
            c = np.searchsorted(cp, p, side="right") - 1
            assert br[pos[p]] == ri[p] and ci[pos[p]] == c
        for c in range(12):
            assert np.all(np.diff(ri[cp[c]:cp[c + 1]]) > 0)


def test_quantile_bit_exact_vs_torch():
    g = torch.Generator().manual_seed(0)
    for n in (16, 1024, 4096, 16384, 65536):
        for q in (0.5, 0.75, 0.85, 0.96, 0.98, 0.99, 0.123, 0.0, 1.0):
            for _ in range(6):
                x = torch.rand(n, generator=g) ** 3
                t = np.float32(torch.quantile(x, q).item())
                assert opat.quantile_threshold(x.numpy(), q) == t


def test_walker_rule_ties_and_guards():
    # all-equal map: every comparison ties -> diagonal moves only; nothing exceeds thresh
    p = np.full((6, 6), 0.25, np.float32)
    assert opat.greedy_paths(p, 0.25).sum() == 0
    # below-threshold cells are walked through but not marked
    m = opat.greedy_paths(p, 0.1)
    # seeds (0,k) walk the diagonal k..: marks (1,k+1),(2,k+2).. ; seeds (k,0) likewise
    want = np.zeros((6, 6), np.uint8)
    for k in range(6):
        for t in range(1, 6 - k):
            want[t, k + t] = 1
            want[k + t, t] = 1
    assert np.array_equal(m, want)
    # D == R falls into the "right/diag" branch (main_conv_ff.py:40,51)
    p = np.zeros((3, 3), np.float32)
    p[1, 0] = 0.5; p[0, 1] = 0.5
    m = opat.greedy_paths(p, 0.1)
    assert m[0, 1] == 1          # seed (0,0): D == R -> R > G -> right
    # zero map: only the forced diagonal remains
    mat, _, _ = opat.discover_block_mask(np.zeros((64, 64), np.float32), 32, 0.9)
    assert np.array_equal(mat, np.eye(2, dtype=np.uint8))


def test_topk_matches_reference():
    z, cases = _load("topk_reference.npz")
    for c in cases:
        seed, L, bs = [int(x) for x in z[c + "/meta"]]
        nb = L // bs
        A = synthetic.structured_map(seed, L).numpy()
        gold = np.unpackbits(z[c + "/mat"])[:nb * nb].reshape(nb, nb)
        mat, _ = opat.discover_block_mask_topk(A, bs, float(z[c + "/density"]))
        assert np.array_equal(mat, gold)


def test_stack_shape():
    m = opat.stack_for_reference([np.eye(4), np.eye(4)])
    assert m.shape == (4, 2, 4, 4) and m.dtype == np.float32
