"""Edge cases of the tcgen05 engine (bf16, native tiles) against the oracle: rows that need several
chunks, rows with one block, full masks, key padding with fully padded tails, 32-wide masks on
super-blocks, and the bounded-wait failure path (which faults nothing)."""
import numpy as np
import pytest
import torch

from oracle import attention as oatt
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu
REL = 2e-2


def cfg(B, H, L, d, bs):
    return {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
            "transformer_dim": H * d, "task": "t"}


def rel(a, b):
    b = b.float().cpu()
    return float((a.detach().float().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def check(B, H, L, d, bs, mat, keypad=None, seed=5):
    """Both backward paths of the engine: tiles rebuilt on chip from the log-sum-exp (the default), and the
    kernels that read stored P tiles and write dS tiles (spion_attn_backward_ex)."""
    for recompute in (True, False):
        check_one(B, H, L, d, bs, mat, keypad, seed, recompute)


def check_one(B, H, L, d, bs, mat, keypad, seed, recompute):
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    Q, K, V, dO = [t.to(torch.bfloat16) for t in synthetic.qkv(seed, B, H, L, d)]
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.bfloat16, keypad=keypad is not None,
                               engine=_lib.ENGINE_TCGEN05, recompute=recompute)
    assert mod.fused and mod.recompute == recompute
    q = Q.cuda().requires_grad_(True); k = K.cuda().requires_grad_(True); v = V.cuda().requires_grad_(True)
    out, P = mod(q, k, v, None if keypad is None else keypad.cuda(), torch.as_tensor(mat).cuda())
    out.backward(dO.cuda())
    torch.cuda.synchronize()
    mod.check_device_status()
    O, Pd, gQ, gK, gV = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, bs, keypad, dO.float())
    want_tiles = torch.as_tensor(oatt.block_values_from_dense(Pd.numpy(), mat, bs))
    assert rel(out, O) <= REL
    assert rel(P.view(B * H, -1, bs, bs), want_tiles) <= REL
    assert rel(q.grad, gQ) <= REL and rel(k.grad, gK) <= REL and rel(v.grad, gV) <= REL


@pytest.mark.parametrize("d", [32, 64])
def test_rows_of_every_length(d):
    """Block rows with 1, 2, 3, 4 (one chunk) and 5..9 blocks (streamed chunks) in one mask."""
    nb = 10
    mat = np.eye(nb, dtype=np.uint8)
    for r in range(nb):
        mat[r, :min(nb, r)] = 1            # row r has r+1 blocks (last: 10)
    check(1, 2, nb * 64, d, 64, mat)


def test_full_mask_is_dense_attention():
    check(1, 2, 512, 64, 64, np.ones((8, 8), np.uint8))


def test_single_column_and_diagonal_only():
    m = np.eye(8, dtype=np.uint8); m[:, 3] = 1
    check(2, 1, 512, 64, 64, m)
    check(2, 1, 512, 32, 64, np.eye(8, dtype=np.uint8))


def test_key_padding_with_fully_padded_tail():
    B, L = 2, 512
    kp = torch.ones(B, L); kp[0, 200:] = 0; kp[1, 64:] = 0        # whole key blocks are padding
    mat = synthetic.band_random_mask(4, 8, 0.5)
    check(B, 2, L, 64, 64, mat, keypad=kp)


@pytest.mark.parametrize("dens", [0.1, 0.6])
def test_blocks_of_32_on_super_blocks(dens):
    mat = synthetic.band_random_mask(11, 16, dens)
    check(1, 2, 512, 64, 32, mat)
    kp = synthetic.key_padding(2, 1, 512)
    check(1, 2, 512, 32, 32, mat, keypad=kp)


def test_bounded_wait_reports_and_context_survives():
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    mod = BlockSparseAttention(cfg(1, 1, 128, 64, 64), dtype=torch.bfloat16)
    rc = _lib.lib.spion_selftest_bounded_wait(mod.handle, 2_000_000)      # about a millisecond
    assert rc == -4, "the wait must give up and be reported as SPION_ERR_TIMEOUT"
    mod.check_device_status()                                              # word was cleared
    check(1, 1, 128, 64, 64, np.ones((2, 2), np.uint8))                    # the GPU context still works


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mean_map_from_tiles_and_dense_via_blocks(dtype):
    from spion_b200.native import DenseViaBlocks
    B, H, L, d, bs = 2, 2, 256, 64, 64
    Q, K, V = [t.to(dtype) for t in synthetic.qkv(9, B, H, L, d, n=3)]
    mod = DenseViaBlocks(cfg(B, H, L, d, bs), dtype=dtype)
    out, P = mod(Q.cuda(), K.cuda(), V.cuda())
    A = mod.mean_attention_map(P)
    O, Pd = oatt.dense_attention(Q.float(), K.float(), V.float())
    want = Pd.mean(0).mean(0)
    tol = 1e-6 if dtype == torch.float32 else 2e-2 * float(want.max())
    assert float((A.cpu() - want).abs().max()) <= tol
    assert rel(out, O) <= (1e-4 if dtype == torch.float32 else REL)
    # sparse mask: cells outside the mask are exactly zero
    from spion_b200.native import BlockSparseAttention
    mat = synthetic.band_random_mask(3, L // bs, 0.4)
    sp = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=dtype)
    _, Ps = sp(Q.cuda(), K.cuda(), V.cuda(), None, torch.as_tensor(mat).cuda())
    As = sp.mean_attention_map(Ps).cpu()
    M = oatt.expand_mask(mat, bs)
    assert float((As * (1 - M)).abs().max()) == 0.0
    _, Pm = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, bs)
    assert float((As - Pm.mean(0).mean(0)).abs().max()) <= tol


@pytest.mark.parametrize("d,bs", [(64, 64), (32, 64), (64, 32)])
def test_mean_map_rebuilt_from_lse(d, bs):
    """The warm-up map A = mean_bh P from Q, K and the log-sum-exp (no stored probabilities): full mask, with
    key padding, with merged-head operands, and on a sparse 32-wide mask (zero outside the selected blocks)."""
    from spion_b200.native import BlockSparseAttention, DenseViaBlocks, ProbsHandle
    B, H, L = 3, 1, 256                                             # odd number of (b,h) matrices
    Q, K, V = [t.to(torch.bfloat16) for t in synthetic.qkv(13, B, H, L, d, n=3)]
    kp = synthetic.key_padding(6, B, L)
    for keypad in (None, kp):
        mod = DenseViaBlocks(cfg(B, H, L, d, bs), dtype=torch.bfloat16, keypad=keypad is not None)
        out, probs = mod(Q.cuda(), K.cuda(), V.cuda(), None if keypad is None else keypad.cuda())
        assert isinstance(probs, ProbsHandle)
        A = mod.mean_attention_map(probs)
        mod.block.check_device_status()
        O, Pd = oatt.sparse_attention(Q.float(), K.float(), V.float(), np.ones((L // bs, L // bs), np.uint8), bs, keypad)
        want = Pd.mean(0).mean(0)
        assert float((A.cpu() - want).abs().max()) <= 2e-2 * float(want.max())
        assert rel(out, O) <= REL
    # sparse mask, merged-head operands, two heads
    B, H = 2, 2
    Q, K, V = [t.to(torch.bfloat16) for t in synthetic.qkv(14, B, H, L, d, n=3)]
    mat = synthetic.band_random_mask(3, L // bs, 0.4)
    sp = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.bfloat16, return_probs=False)
    merged = [t.cuda().transpose(1, 2).contiguous().transpose(1, 2) for t in (Q, K, V)]
    out, probs = sp(*merged, None, torch.as_tensor(mat).cuda())
    assert isinstance(probs, ProbsHandle) and probs.heads == H
    A = sp.mean_attention_map(probs).cpu()
    sp.check_device_status()
    _, Pm = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, bs)
    want = Pm.mean(0).mean(0)
    assert float((A * (1 - oatt.expand_mask(mat, bs))).abs().max()) == 0.0
    assert float((A - want).abs().max()) <= 2e-2 * float(want.max())
