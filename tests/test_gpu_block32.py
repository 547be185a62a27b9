"""Masks of 32 x 32 blocks with head_dim 64 on the tensor-core engine: the kernels that work on the mask's own
blocks (gathered 128-row operands, transposed products; csrc/tc_b32.cu) against the oracle, and against the
super-block path they replace for the calls that store no probabilities.

What the reference computes for such masks: models/block_attn.cu:453-545 with block_size 32
(config.py: the image task).
"""
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
    b = b.detach().float().cpu()
    return float((a.detach().float().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def run(B, H, L, mat, keypad=None, seed=5, merged=False, path="own"):
    """forward + backward through the public module without stored probabilities (the calls the block-32
    kernels serve); returns (O, dQ, dK, dV) as float CPU tensors and the inputs."""
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    d, bs = 64, 32
    Q, K, V, dO = [t.to(torch.bfloat16) for t in synthetic.qkv(seed, B, H, L, d)]
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.bfloat16, keypad=keypad is not None,
                               engine=_lib.ENGINE_TCGEN05, recompute=True, return_probs=False, block32=path)
    assert mod.fused and mod.recompute

    def prep(t):
        t = t.cuda()
        if merged:                                               # [B, L, H*d] storage seen as [B, H, L, d]
            t = t.transpose(1, 2).contiguous().view(B, L, H * d).view(B, L, H, d).transpose(1, 2)
            assert mod.operand_form(t) == H
        return t.requires_grad_(True)

    q, k, v = prep(Q), prep(K), prep(V)
    out, _ = mod(q, k, v, None if keypad is None else keypad.cuda(), torch.as_tensor(mat).cuda())
    g = dO.cuda()
    if merged:
        g = g.transpose(1, 2).contiguous().transpose(1, 2)
    out.backward(g)
    torch.cuda.synchronize()
    mod.check_device_status()
    return (Q, K, V, dO), [t.detach().float().cpu() for t in (out, q.grad, k.grad, v.grad)]


def check(B, H, L, mat, keypad=None, seed=5, merged=False):
    (Q, K, V, dO), got = run(B, H, L, mat, keypad, seed, merged)
    want = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, 32, keypad, dO.float())
    O, _, gQ, gK, gV = want
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, (O, gQ, gK, gV)):
        assert rel(a, b) <= REL, f"{name}: {rel(a, b):.3e}"


def test_rows_and_columns_of_every_length():
    """Block rows with 1..16 blocks and block columns with 16..1 entries: one to four gathered jobs per unit,
    partially filled last jobs, several jobs per unit in flight."""
    nb = 16
    mat = np.eye(nb, dtype=np.uint8)
    for r in range(nb):
        mat[r, :r] = 1
    check(1, 2, nb * 32, mat)


def test_diagonal_only_and_full_mask():
    check(1, 1, 512, np.eye(16, dtype=np.uint8))
    check(1, 2, 512, np.ones((16, 16), np.uint8))


@pytest.mark.parametrize("dens", [0.1, 0.6])
def test_random_masks(dens):
    check(2, 2, 512, synthetic.band_random_mask(11, 16, dens))


def test_many_units_per_cta():
    """More units than the persistent grid holds CTAs: every CTA walks several units (accumulator and
    small-operand buffers alternate, records of following units are requested ahead)."""
    check(4, 8, 2048, synthetic.band_random_mask(7, 64, 0.05), seed=9)


def test_key_padding():
    kp = synthetic.key_padding(2, 2, 512)
    kp[1, 64:] = 0                                               # whole key blocks are padding
    check(2, 2, 512, synthetic.band_random_mask(3, 16, 0.4), keypad=kp)


def test_lines_without_blocks():
    """A mask need not contain its diagonal when the caller sets it by hand: block rows without a selected
    block give zero output rows (and the denominator of the non-selected keys), block columns without an
    entry give zero dK and dV rows."""
    nb = 8
    mat = np.zeros((nb, nb), np.uint8)
    mat[0, 1] = mat[1, 1] = mat[2, 5] = mat[5, 2] = mat[7, 1] = 1          # rows 3, 4, 6 and columns 0, 3, 4, 6, 7 are empty
    check(1, 2, nb * 32, mat)


def test_merged_head_operands():
    mat = synthetic.band_random_mask(9, 16, 0.5)
    (_, _, _, _), packed = run(2, 3, 512, mat, seed=21)
    (Q, K, V, dO), merged = run(2, 3, 512, mat, seed=21, merged=True)
    for name, a, b in zip(("O", "dQ", "dK", "dV"), packed, merged):
        assert torch.equal(a, b), f"{name}: merged-head operands give different numbers than packed ones"


@pytest.mark.parametrize("dens,own", [(0.02, False), (0.3, True)])
def test_path_chosen_per_mask(dens, own):
    """With block32="auto" a mask that is little more than its diagonal band (about two blocks per row) stays on
    the super-blocks, a mask with fuller rows runs on its own blocks; both give the oracle's numbers, and the
    choice shows in the kernels' stage timers (the two paths report different stage sets)."""
    B, H, L = 2, 2, 2048
    mat = synthetic.band_random_mask(2056, L // 32, dens)
    fill = mat.sum() / np.ceil(mat.sum(1) / 4).sum()
    assert (fill >= 2.8) == own, fill
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    probe = BlockSparseAttention(cfg(B, H, L, 64, 32), dtype=torch.bfloat16, engine=_lib.ENGINE_TCGEN05)
    probe.set_mask(torch.as_tensor(mat).cuda())
    assert _lib.lib.spion_block32_path_in_use(probe.handle) == (1 if own else 2)
    (Q, K, V, dO), got = run(B, H, L, mat, seed=17, path="auto")
    O, _, gQ, gK, gV = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, 32, None, dO.float())
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, (O, gQ, gK, gV)):
        assert rel(a, b) <= REL, f"{name}: {rel(a, b):.3e}"


def test_agrees_with_the_super_block_path():
    """The same call with stored probabilities runs on 64-wide super-blocks (the path that also serves
    head_dim 32): outputs and gradients of the two paths agree to bf16 rounding."""
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    B, H, L, d, bs = 2, 2, 1024, 64, 32
    mat = synthetic.band_random_mask(13, L // bs, 0.2)
    (Q, K, V, dO), own = run(B, H, L, mat, seed=31)
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.bfloat16, engine=_lib.ENGINE_TCGEN05, recompute=False)
    q, k, v = [t.cuda().requires_grad_(True) for t in (Q, K, V)]
    out, P = mod(q, k, v, None, torch.as_tensor(mat).cuda())
    out.backward(dO.cuda())
    torch.cuda.synchronize()
    mod.check_device_status()
    for name, a, b in zip(("O", "dQ", "dK", "dV"), own, (out, q.grad, k.grad, v.grad)):
        assert rel(a, b) <= REL, f"{name}: {rel(a, b):.3e}"


def test_path_argument_is_checked():
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    mod = BlockSparseAttention(cfg(1, 1, 256, 64, 32), dtype=torch.bfloat16)
    assert _lib.lib.spion_set_block32_path(mod.handle, 3) == -1          # SPION_ERR_ARG
    assert _lib.lib.spion_set_block32_path(mod.handle, 2) == 0
    mod.set_mask(torch.ones(8, 8, dtype=torch.uint8, device="cuda"))
    assert _lib.lib.spion_block32_path_in_use(mod.handle) == 2
    with pytest.raises(KeyError):
        BlockSparseAttention(cfg(1, 1, 256, 64, 32), dtype=torch.bfloat16, block32="fastest")
