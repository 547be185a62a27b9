"""The plain-C restatement (oracle/spion_oracle.c) against the reference's golden fixtures and against the numpy /
torch restatement: integer results, pooled map and threshold bit for bit, the attention step within fp32 rounding."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from oracle import c_oracle
from oracle import csr as ocsr
from oracle import pattern as opat
from spion_b200 import synthetic

pytestmark = pytest.mark.skipif(c_oracle.load() is None, reason="no C compiler and no prebuilt oracle library")
GOLD = os.path.join(os.path.dirname(__file__), "golden")
PAT = np.load(os.path.join(GOLD, "pattern_reference.npz"))
PAT_CASES = sorted({k.split("/")[0] for k in PAT.files})
TOPK = np.load(os.path.join(GOLD, "topk_reference.npz"))
TOPK_CASES = sorted({k.split("/")[0] for k in TOPK.files})


def _map(meta):
    seed, L, bs, F, ck, mk = [int(x) for x in meta]
    if mk == 0:
        Q, K = synthetic.qkv(seed, 2, 2, L, 32, n=2)
        A = synthetic.mean_attention_map(Q, K)
    else:
        A = synthetic.structured_map(seed, L)
    return A.numpy(), L, bs, F, ck


@pytest.mark.parametrize("case", PAT_CASES)
def test_c_mask_matches_reference_fixture(case):
    A, L, bs, F, ck = _map(PAT[case + "/meta"])
    nb = L // bs
    gold = np.unpackbits(PAT[case + "/mat"])[:nb * nb].reshape(nb, nb)
    q = float(PAT[case + "/q"])
    mat_c, thr_c, pooled_c = c_oracle.discover(A, bs, q, F, ck)
    mat_n, thr_n, pooled_n = opat.discover_block_mask(A, bs, q, F, ck, float_path="fixed")
    assert np.array_equal(pooled_c.view(np.uint32), pooled_n.view(np.uint32)), "pooled map differs in some bit"
    assert np.float32(thr_c).tobytes() == np.float32(thr_n).tobytes()
    assert np.array_equal(mat_c, mat_n) and np.array_equal(mat_c, gold)
    # CSR of the mask: the reference's torch lines (hashed in the fixture), numpy and C agree
    sm, off, col, nnz = c_oracle.element_csr(gold, bs, 1)
    assert nnz == int(PAT[case + "/nnz"])
    assert hashlib.sha256(np.concatenate([sm, off, col]).tobytes()).digest() == PAT[case + "/csr_sha"].tobytes()
    rp, ci, br, cp, ri, pos = c_oracle.block_csr(gold)
    rp_n, ci_n, br_n = ocsr.block_csr(gold)
    cp_n, ri_n, pos_n = ocsr.block_csc(gold)
    for a, b in ((rp, rp_n), (ci, ci_n), (br, br_n), (cp, cp_n), (ri, ri_n), (pos, pos_n)):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("case", TOPK_CASES)
def test_c_topk_variant(case):
    seed, L, bs = [int(x) for x in TOPK[case + "/meta"]]
    nb = L // bs
    A = synthetic.structured_map(seed, L).numpy()
    density = float(TOPK[case + "/density"])
    gold = np.unpackbits(TOPK[case + "/mat"])[:nb * nb].reshape(nb, nb)
    mat_c, _, pooled_c = c_oracle.discover(A, bs, density, select="topk")
    mat_n, pooled_n = opat.discover_block_mask_topk(A, bs, density)
    assert np.array_equal(pooled_c.view(np.uint32), pooled_n.view(np.uint32))
    assert np.array_equal(mat_c, mat_n) and np.array_equal(mat_c, gold)


def test_c_elementcsr_repeat_and_ragged_rows():
    mat = np.zeros((5, 5), np.uint8)
    mat[0, :] = 1; mat[2, 3] = 1; mat[4, 0] = 1; mat[4, 4] = 1          # full row, single block, empty rows
    for rep in (1, 3):
        got = c_oracle.element_csr(mat, 4, rep)
        want = ocsr.element_csr(mat, 4, rep)
        assert got[3] == want[3]
        for a, b in zip(got[:3], want[:3]):
            assert np.array_equal(a, b)


@pytest.mark.parametrize("B,H,L,d,bs,dens,kpm", [(2, 2, 128, 32, 32, 0.5, False), (1, 3, 256, 64, 64, 0.4, False),
                                                 (2, 1, 256, 32, 32, 0.3, True)])
def test_c_attention_step_matches_torch_oracle(B, H, L, d, bs, dens, kpm):
    Q, K, V, dO = synthetic.qkv(5 + L, B, H, L, d)
    mat = synthetic.band_random_mask(L + 1, L // bs, dens)
    kp = synthetic.key_padding(3, B, L) if kpm else None
    pen = None
    if kpm:
        pen = (1e6 * (1 - kp))[:, None, :].expand(B, H, L).reshape(B * H, L).numpy()
    O, P, dQ, dK, dV = c_oracle.attention_step(Q.numpy(), K.numpy(), V.numpy(), mat, bs, dO.numpy(), pen)
    wO, wP, wQ, wK, wV = oatt.sparse_attention(Q, K, V, mat, bs, kp, dO)
    wP = oatt.csr_values_from_dense(wP.numpy(), mat, bs)
    for got, want, name in ((O, wO, "O"), (P, wP, "P"), (dQ, wQ, "dQ"), (dK, wK, "dK"), (dV, wV, "dV")):
        err = float(np.abs(got - np.asarray(want)).max())
        assert err <= 2e-5, f"{name}: {err}"
    # forward only gives the same bits
    O2, P2 = c_oracle.attention_step(Q.numpy(), K.numpy(), V.numpy(), mat, bs, penalty=pen)
    assert np.array_equal(O2, O) and np.array_equal(P2, P)


def test_c_attention_row_emulation_small():
    B, H, L, d, bs = 1, 2, 64, 32, 32
    Q, K, V, dO = synthetic.qkv(9, B, H, L, d)
    mat = np.array([[1, 0], [1, 1]], np.uint8)
    O, P, dQ, dK, dV = c_oracle.attention_step(Q.numpy(), K.numpy(), V.numpy(), mat, bs, dO.numpy())
    Pv, wO, wQ, wK, wV = oatt.sparse_attention_rowwise(Q.numpy(), K.numpy(), V.numpy(), mat, bs, None, dO.numpy())
    wP = np.stack([np.concatenate(rows) for rows in Pv])
    for got, want in ((O, wO), (P, wP), (dQ, wQ), (dK, wK), (dV, wV)):
        assert float(np.abs(got - want).max()) <= 5e-6


LARGE = np.load(os.path.join(GOLD, "pattern_reference_large.npz"))
LARGE_CASES = sorted({k.split("/")[0] for k in LARGE.files})


@pytest.mark.parametrize("case", LARGE_CASES)
def test_c_mask_at_the_largest_block_counts(case):
    """nb = 256 and nb = 512 (the largest of the kernel sweep): the reference's own walkers against the C
    restatement (and, at nb = 256, the numpy one too; at nb = 512 that one takes minutes)."""
    A, L, bs, F, ck = _map(LARGE[case + "/meta"])
    assert hashlib.sha256(np.ascontiguousarray(A).tobytes()).digest() == LARGE[case + "/sha"].tobytes()
    nb = L // bs
    gold = np.unpackbits(LARGE[case + "/mat"])[:nb * nb].reshape(nb, nb)
    q = float(LARGE[case + "/q"])
    mat_c, thr_c, pooled_c = c_oracle.discover(A, bs, q, F, ck)
    assert np.array_equal(mat_c, gold)
    # the reference's float stages sum in another order: the threshold agrees to rounding, the mask exactly
    assert abs(float(thr_c) - float(LARGE[case + "/thresh"])) <= 2e-5 * abs(float(thr_c))
    sm, off, col, nnz = c_oracle.element_csr(gold, bs, 1)
    assert nnz == int(LARGE[case + "/nnz"])
    assert hashlib.sha256(np.concatenate([sm, off, col]).tobytes()).digest() == LARGE[case + "/csr_sha"].tobytes()
    if nb <= 256:
        mat_n, thr_n, pooled_n = opat.discover_block_mask(A, bs, q, F, ck, float_path="fixed")
        assert np.array_equal(pooled_c.view(np.uint32), pooled_n.view(np.uint32))
        assert np.float32(thr_c).tobytes() == np.float32(thr_n).tobytes() and np.array_equal(mat_n, gold)
