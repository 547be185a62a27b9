"""GPU parity of pattern discovery and CSR construction (integer outputs: bit-exact)."""
import os

import numpy as np
import pytest
import torch

from oracle import csr as ocsr
from oracle import pattern as opat
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _pattern_mod():
    from spion_b200 import pattern
    return pattern


def _map(meta):
    seed, L, bs, F, ck, mk = [int(x) for x in meta]
    if mk == 0:
        Q, K = synthetic.qkv(seed, 2, 2, L, 32, n=2)
        A = synthetic.mean_attention_map(Q, K)
    else:
        A = synthetic.structured_map(seed, L)
    return A, L, bs, F, ck


def _check_structure(p, mat):
    rp, ci, br = ocsr.block_csr(mat)
    cp, ri, pos = ocsr.block_csc(mat)
    assert p.nnzb == int(mat.sum())
    assert np.array_equal(p.row_ptr.cpu().numpy(), rp)
    assert np.array_equal(p.col_idx.cpu().numpy(), ci)
    assert np.array_equal(p.blk_row.cpu().numpy(), br)
    assert np.array_equal(p.col_ptr.cpu().numpy(), cp)
    assert np.array_equal(p.row_idx.cpu().numpy(), ri)
    assert np.array_equal(p.csc_pos.cpu().numpy(), pos)


PAT = np.load(os.path.join(GOLD, "pattern_reference.npz"))
CASES = sorted({k.split("/")[0] for k in PAT.files})


@pytest.mark.parametrize("case", CASES)
def test_discovery_matches_reference_mask_and_oracle_bits(case):
    pattern = _pattern_mod()
    A, L, bs, F, ck = _map(PAT[case + "/meta"])
    nb = L // bs
    q = float(PAT[case + "/q"])
    gold = np.unpackbits(PAT[case + "/mat"])[:nb * nb].reshape(nb, nb)
    p = pattern.discover_pattern(A.cuda(), bs, q, conv="diag" if ck == 0 else "box", F=F)
    mat = p.mat.cpu().numpy()
    # the reference's own mask (made by its flood_fill on the CPU)
    assert np.array_equal(mat, gold)
    # float stages: same bits as the fixed-order oracle
    o_mat, o_thr, o_pooled = opat.discover_block_mask(A.numpy(), bs, q, F, ck, float_path="fixed")
    assert np.array_equal(p.pooled.cpu().numpy(), o_pooled)
    assert np.float32(p.thresh.item()) == o_thr
    _check_structure(p, gold)
    # element CSR as the reference's torch lines build it
    sm, off, col, nnz = p.element_csr(repeat=2)
    o_sm, o_off, o_col, o_nnz = ocsr.element_csr(gold, bs, 2)
    assert nnz == o_nnz == int(PAT[case + "/nnz"])
    assert np.array_equal(sm.cpu().numpy(), o_sm)
    assert np.array_equal(off.cpu().numpy(), o_off)
    assert np.array_equal(col.cpu().numpy(), o_col)


def test_topk_variant_matches_reference():
    pattern = _pattern_mod()
    z = np.load(os.path.join(GOLD, "topk_reference.npz"))
    for c in sorted({k.split("/")[0] for k in z.files}):
        seed, L, bs = [int(x) for x in z[c + "/meta"]]
        nb = L // bs
        A = synthetic.structured_map(seed, L)
        gold = np.unpackbits(z[c + "/mat"])[:nb * nb].reshape(nb, nb)
        p = pattern.discover_pattern(A.cuda(), bs, float(z[c + "/density"]), select="topk")
        assert np.array_equal(p.mat.cpu().numpy(), gold)
        _check_structure(p, gold)


@pytest.mark.parametrize("L,bs,F,kind", [(256, 32, 31, 0), (256, 64, 31, 0), (512, 32, 3, 1), (512, 64, 5, 1),
                                         (256, 32, 1, 0), (2048, 32, 31, 0)])
def test_random_maps_bit_exact_vs_oracle(L, bs, F, kind):
    pattern = _pattern_mod()
    for seed in range(3):
        g = torch.Generator().manual_seed(100 + seed)
        A = torch.softmax(torch.randn(L, L, generator=g) * 2.0, dim=-1)
        for q in (0.5, 0.9):
            p = pattern.discover_pattern(A.cuda(), bs, q, conv="diag" if kind == 0 else "box", F=F)
            o_mat, o_thr, o_pooled = opat.discover_block_mask(A.numpy(), bs, q, F, kind)
            assert np.array_equal(p.pooled.cpu().numpy(), o_pooled)
            assert np.float32(p.thresh.item()) == o_thr
            assert np.array_equal(p.mat.cpu().numpy(), o_mat)


def test_edge_cases():
    pattern = _pattern_mod()
    # zero map: only the forced diagonal
    p = pattern.discover_pattern(torch.zeros(128, 128).cuda(), 32, 0.9)
    assert np.array_equal(p.mat.cpu().numpy(), np.eye(4, dtype=np.uint8)) and p.nnzb == 4
    # constant map: every comparison ties, walkers go diagonally, nothing exceeds the threshold
    p = pattern.discover_pattern(torch.full((128, 128), 0.01).cuda(), 32, 0.5)
    o, _, _ = opat.discover_block_mask(np.full((128, 128), 0.01, np.float32), 32, 0.5)
    assert np.array_equal(p.mat.cpu().numpy(), o)
    # one block
    p = pattern.discover_pattern(torch.rand(32, 32).cuda(), 32, 0.5)
    assert p.nnzb == 1 and p.row_ptr.tolist() == [0, 1]
    # ragged length is refused
    with pytest.raises(ValueError):
        pattern.discover_pattern(torch.rand(100, 100).cuda(), 32, 0.5)
    # largest supported block grid: L=16384, bs=32 -> nb=512 (structure only; the map would be 1 GiB)
    mat = synthetic.band_random_mask(1, 512, 0.02)
    ps = pattern.pattern_from_mask(torch.as_tensor(mat).cuda(), 32)
    _check_structure(ps, mat)
    # full and empty-off-diagonal masks
    for m in (np.ones((8, 8), np.uint8), np.eye(8, dtype=np.uint8)):
        _check_structure(pattern.pattern_from_mask(torch.as_tensor(m).cuda(), 64), m)


def test_mean_attention_map_both_storages():
    pattern = _pattern_mod()
    g = torch.Generator().manual_seed(3)
    attn = torch.rand(3, 2, 128, 128, generator=g)
    want = attn.mean(0).mean(0)
    got = pattern.mean_attention_map(attn.cuda().contiguous())
    np.testing.assert_allclose(got.cpu().numpy(), want.numpy(), rtol=1e-6, atol=1e-7)
    got_t = pattern.mean_attention_map(attn.permute(0, 1, 3, 2).contiguous().cuda(), transposed_storage=True)
    np.testing.assert_allclose(got_t.cpu().numpy(), want.numpy(), rtol=1e-6, atol=1e-7)


def test_discover_layers_reference_form():
    pattern = _pattern_mod()
    cfg = {"block_size": 32, "max_seq_len": 256, "threshold": 0.8, "num_layers": 2}
    maps = [synthetic.structured_map(s, 256).cuda() for s in (1, 2)]
    mat_lst, pats = pattern.discover_layers(maps, cfg)
    assert mat_lst.shape == (4, 2, 8, 8) and mat_lst.dtype == torch.float32
    for l in range(2):
        o, _, _ = opat.discover_block_mask(maps[l].cpu().numpy(), 32, 0.8)
        assert np.array_equal(mat_lst[0][l].cpu().numpy(), o.astype(np.float32))


LARGE = np.load(os.path.join(GOLD, "pattern_reference_large.npz"))


@pytest.mark.parametrize("case", sorted({k.split("/")[0] for k in LARGE.files}))
def test_discovery_at_the_largest_block_counts(case):
    """nb = 256 and nb = 512 (L = 16384 at block 64 / 32): the masks the reference's own walkers produced,
    reproduced by the kernels bit for bit, with the CSR / CSC and the element CSR that belong to them."""
    import hashlib
    pattern = _pattern_mod()
    A, L, bs, F, ck = _map(LARGE[case + "/meta"])
    assert hashlib.sha256(np.ascontiguousarray(A.numpy()).tobytes()).digest() == LARGE[case + "/sha"].tobytes()
    nb = L // bs
    gold = np.unpackbits(LARGE[case + "/mat"])[:nb * nb].reshape(nb, nb)
    q = float(LARGE[case + "/q"])
    p = pattern.discover_pattern(A.cuda(), bs, q, conv="diag" if ck == 0 else "box", F=F)
    assert np.array_equal(p.mat.cpu().numpy(), gold)
    assert abs(float(p.thresh.item()) - float(LARGE[case + "/thresh"])) <= 2e-5 * abs(float(p.thresh.item()))
    _check_structure(p, gold)
    sm, off, col, nnz = p.element_csr(repeat=1)
    assert nnz == int(LARGE[case + "/nnz"])
    got = np.concatenate([sm.cpu().numpy(), off.cpu().numpy(), col.cpu().numpy()])
    assert hashlib.sha256(got.tobytes()).digest() == LARGE[case + "/csr_sha"].tobytes()
