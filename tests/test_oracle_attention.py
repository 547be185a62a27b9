"""Pin the attention oracle: dense case against the reference's SoftmaxAttention outputs,
sparse closed form against the statement-by-statement emulation of the reference kernels."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from spion_b200 import synthetic

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_dense_matches_reference_softmax_attention():
    z = np.load(os.path.join(GOLD, "dense_attention_reference.npz"))
    for c in sorted({k.split("/")[0] for k in z.files}):
        seed, B, H, L, d = [int(x) for x in z[c + "/meta"]]
        Q, K, V = synthetic.qkv(seed, B, H, L, d, n=3)
        kp = synthetic.key_padding(seed, B, L)
        O, P = oatt.dense_attention(Q, K, V, kp)
        np.testing.assert_allclose(O.numpy(), z[c + "/out"], atol=2e-6, rtol=1e-5)
        np.testing.assert_allclose(P[:, :, ::7, ::5].numpy(), z[c + "/attn_sample"], atol=1e-7, rtol=1e-5)
        np.testing.assert_allclose(P.sum(-1).numpy(), z[c + "/attn_rowsum"], atol=1e-5)


@pytest.mark.parametrize("kpm", [False, True])
@pytest.mark.parametrize("bs,d", [(32, 32), (64, 64)])
def test_closed_form_equals_kernel_statement_emulation(bs, d, kpm):
    B, H, nb = 2, 2, 4
    L = nb * bs
    Q, K, V, dO = synthetic.qkv(5 + bs + d, B, H, L, d)
    mat = synthetic.band_random_mask(3, nb, 0.45)
    kp = synthetic.key_padding(9, B, L) if kpm else None
    O, P, dQ, dK, dV = oatt.sparse_attention(Q, K, V, mat, bs, kp, dO)
    rows, O2, dQ2, dK2, dV2 = oatt.sparse_attention_rowwise(Q.numpy(), K.numpy(), V.numpy(), mat, bs,
                                                            None if kp is None else kp.numpy(), dO.numpy())
    np.testing.assert_allclose(O.numpy(), O2, atol=2e-6)
    np.testing.assert_allclose(dQ.numpy(), dQ2, atol=5e-6)
    np.testing.assert_allclose(dK.numpy(), dK2, atol=5e-6)
    np.testing.assert_allclose(dV.numpy(), dV2, atol=5e-6)
    vals = oatt.csr_values_from_dense(P.numpy(), mat, bs)
    flat = np.concatenate([np.concatenate(r) for r in rows]).reshape(B * H, -1)
    np.testing.assert_allclose(vals, flat, atol=5e-7, rtol=1e-5)
    # rows do not sum to one: the non-selected keys keep their share of the denominator
    assert float(P.sum(-1).max()) < 1.0


def test_value_layout_helpers():
    bs, nb = 4, 3
    mat = np.array([[1, 0, 1], [0, 1, 0], [1, 1, 1]], np.uint8)
    L = nb * bs
    P = torch.arange(L * L, dtype=torch.float32).reshape(1, 1, L, L)
    v = oatt.csr_values_from_dense(P.numpy(), mat, bs)
    assert v.shape == (1, int(mat.sum()) * bs * bs)
    assert v[0, 0] == 0 and v[0, bs] == 2 * bs            # row 0: block col 0 then block col 2
    t = oatt.block_values_from_dense(P.numpy(), mat, bs)
    assert t.shape == (1, int(mat.sum()), bs, bs)
    assert t[0, 1, 0, 0] == 2 * bs and t[0, 2, 0, 0] == bs * L + bs


def test_blockwise_fp64_oracle_matches_dense_masked_closed_form():
    """The block-row oracle used for the large GPU parity cases, against the dense-masked closed form in
    fp64 (with and without key padding, block 32 and 64, an empty-looking row of one block)."""
    for seed, (B, H, L, d, bs, dens, kpm) in enumerate([(1, 2, 256, 32, 32, 0.3, False), (2, 1, 256, 64, 64, 0.5, True),
                                                        (1, 1, 512, 64, 32, 0.1, False)]):
        Q, K, V, dO = synthetic.qkv(40 + seed, B, H, L, d)
        mat = synthetic.band_random_mask(seed, L // bs, dens)
        kp = synthetic.key_padding(seed, B, L) if kpm else None
        O, P, gQ, gK, gV = oatt.sparse_attention(Q, K, V, mat, bs, kp, dO, dtype=torch.float64)
        tiles = oatt.block_values_from_dense(P.numpy(), mat, bs)
        for b in range(B):
            for h in range(H):
                o, pt, dq, dk, dv = oatt.sparse_attention_blockwise(Q[b, h].numpy(), K[b, h].numpy(), V[b, h].numpy(), mat, bs,
                                                                     None if kp is None else kp[b].numpy(), dO[b, h].numpy())
                assert np.abs(o - O[b, h].numpy()).max() < 1e-12
                assert np.abs(pt - tiles[b * H + h]).max() < 1e-13
                assert np.abs(dq - gQ[b, h].numpy()).max() < 1e-12
                assert np.abs(dk - gK[b, h].numpy()).max() < 1e-12
                assert np.abs(dv - gV[b, h].numpy()).max() < 1e-12
