"""Stand-alone sparse row softmax on block tiles (spion_softmax_forward_ex / spion_softmax_backward_ex) against a
torch fp64 restatement of the reference's kernels (models/block_attn.cu:33-130, key padding as
models/block_attn_mask.cu:88-140):

    v = S * scale - keypad[col];  m = max(floor, max_row v);  Z = sum_row exp(v - m) + (L - n_row) exp(-m)
    P = exp(v - m) / Z;           dS = (dP * P - P * sum_row(dP * P)) * scale

with floor = -100 without key padding and 0 with it.  Masks are chosen so that rows of every kind occur: empty block
rows, rows short enough to stay in registers, rows that take the multi-pass loops, odd block counts of 32-wide
blocks.  Tolerances: fp32 tiles 2e-6 absolute (P <= 1), bf16 tiles 1e-2 relative to the largest value.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def cfg(B, H, L, d, bs):
    return {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
            "transformer_dim": H * d, "task": "t"}


def mask_with_rows(nb, counts, seed):
    """[nb, nb] mask whose block row r selects counts[r % len(counts)] blocks (capped at nb), random columns."""
    rng = np.random.default_rng(seed)
    mat = np.zeros((nb, nb), np.uint8)
    for r in range(nb):
        n = min(nb, counts[r % len(counts)])
        mat[r, rng.choice(nb, size=n, replace=False)] = 1
    return mat


def reference(S, dP, mat, bs, L, scale, keypad):
    """S, dP: [BH, nnzb, bs, bs] float64 tiles in CSR block order; returns P and dS in the same layout."""
    BH = S.shape[0]
    P = torch.zeros_like(S)
    dS = torch.zeros_like(S)
    floor = 0.0 if keypad is not None else -100.0
    rows, cols = np.nonzero(mat)                                    # row-major = CSR block order
    for r in range(mat.shape[0]):
        ids = np.nonzero(rows == r)[0]
        if len(ids) == 0:
            continue
        v = S[:, ids] * scale                                       # [BH, n, bs(i), bs(j)]
        if keypad is not None:
            kp = torch.stack([keypad[:, c * bs:(c + 1) * bs] for c in cols[ids]], 1)    # [BH, n, bs(j)]
            v = v - kp[:, :, None, :]
        m = v.amax(dim=(1, 3), keepdim=True).clamp_min(floor)
        e = torch.exp(v - m)
        Z = e.sum(dim=(1, 3), keepdim=True) + (L - len(ids) * bs) * torch.exp(-m)
        p = e / Z
        t = dP[:, ids] * p
        P[:, ids] = p
        dS[:, ids] = (t - p * t.sum(dim=(1, 3), keepdim=True)) * scale
    return P, dS


@pytest.mark.parametrize("bs,counts,dtype,with_keypad", [
    (64, [1, 3, 4, 5, 0, 9, 2, 16], torch.float32, False),
    (64, [2, 8, 1, 12, 4, 0, 6, 3], torch.bfloat16, False),
    (32, [1, 3, 8, 9, 0, 17, 5, 32], torch.float32, False),
    (32, [7, 2, 15, 16, 1, 0, 21, 4], torch.bfloat16, True),
    (64, [3, 0, 5, 11, 2, 8, 1, 4], torch.float32, True),
    (16, [1, 4, 0, 9, 2], torch.float32, False),                    # other block sizes: one warp per row
])
def test_softmax_rows_match_restatement(bs, counts, dtype, with_keypad):
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    ptr = _lib.ptr
    lib = _lib.lib
    B, H, L, d = 2, 2, 1024 if bs != 16 else 256, 64
    nb = L // bs
    mat = mask_with_rows(nb, counts, seed=bs + len(counts))
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=dtype, keypad=with_keypad, engine=_lib.ENGINE_SIMT)
    nnzb = mod.set_mask(torch.as_tensor(mat))
    assert nnzb == int(mat.sum())
    g = torch.Generator().manual_seed(11)
    S = (torch.randn(B * H, nnzb, bs, bs, generator=g) * 6.0).cuda()
    dP = torch.randn(B * H, nnzb, bs, bs, generator=g).cuda()
    keypad = None
    if with_keypad:
        keypad = torch.zeros(B * H, L)
        keypad[:, L - 100:] = 1e9                                   # padded keys (models/block_attn_mask.cu:105)
        keypad = keypad.cuda()
    P = torch.full((B * H, nnzb, bs, bs), float("nan"), dtype=dtype, device="cuda")
    dS = torch.full_like(P, float("nan"))
    _lib.check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
    _lib.check(lib.spion_softmax_forward_ex(mod.handle, ptr(S), ptr(keypad) if with_keypad else None, ptr(P)),
               "spion_softmax_forward_ex")
    _lib.check(lib.spion_softmax_backward_ex(mod.handle, ptr(dP), ptr(P), ptr(dS)), "spion_softmax_backward_ex")
    torch.cuda.synchronize()
    scale = 1.0 / np.sqrt(d)
    # the backward is checked on the probabilities the forward produced (rounded to the tile dtype)
    wantP, _ = reference(S.double().cpu(), dP.double().cpu(), mat, bs, L, scale, None if keypad is None else keypad.double().cpu())
    gotP = P.double().cpu()
    assert torch.isfinite(gotP).all()
    tolP = 2e-6 if dtype == torch.float32 else 4e-3                 # bf16: half an ulp of values <= 1
    assert float((gotP - wantP).abs().max()) <= tolP
    t = dP.double().cpu() * gotP
    rows, _ = np.nonzero(mat)
    want_dS = torch.zeros_like(gotP)
    for r in range(nb):
        ids = np.nonzero(rows == r)[0]
        if len(ids):
            want_dS[:, ids] = (t[:, ids] - gotP[:, ids] * t[:, ids].sum(dim=(1, 3), keepdim=True)) * scale
    got_dS = dS.double().cpu()
    assert torch.isfinite(got_dS).all()
    ref_max = float(want_dS.abs().max())
    tol = 2e-6 if dtype == torch.float32 else 1e-2 * ref_max
    assert float((got_dS - want_dS).abs().max()) <= tol


def test_softmax_rows_in_place_fp32():
    """fp32 tiles: P may be the array S was read from (the reference's kernels work in place)."""
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    ptr = _lib.ptr
    lib = _lib.lib
    B, H, L, d, bs = 1, 2, 1024, 64, 64
    mat = mask_with_rows(L // bs, [2, 5, 12, 1], seed=3)
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.float32, engine=_lib.ENGINE_SIMT)
    nnzb = mod.set_mask(torch.as_tensor(mat))
    S = (torch.randn(B * H, nnzb, bs, bs, generator=torch.Generator().manual_seed(2)) * 4.0).cuda()
    out = torch.empty_like(S)
    _lib.check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
    _lib.check(lib.spion_softmax_forward_ex(mod.handle, ptr(S), None, ptr(out)))
    work = S.clone()
    _lib.check(lib.spion_softmax_forward_ex(mod.handle, ptr(work), None, ptr(work)))
    torch.cuda.synchronize()
    assert torch.equal(work, out)
