"""The no-allocation forward (spion_attn_forward_static) against the ordinary native forward.

Who needs it: hosts that may not call cudaMalloc where they run attention (a plugin in a
process whose GPU memory is already budgeted, a latency-critical loop).  The entry point keeps
its fp32 score scratch in an array inside the library, so this test hands it inputs, outputs
and the block CSR only, twice in a row with different inputs (the array keeps the first call's
contents), and expects the same P and O as spion_attn_forward_ex with caller scratch.
Collected last on purpose: if it fails, every other test has already run.
"""
import numpy as np
import pytest
import torch

from spion_b200 import synthetic

pytestmark = pytest.mark.gpu


def _run_pair(dtype, seed, B, H, L, d, bs, mat):
    from spion_b200 import _lib
    from spion_b200._lib import check, lib, ptr
    from spion_b200.native import BlockSparseAttention
    from spion_b200.pattern import pattern_from_mask
    cfg = {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
           "transformer_dim": H * d, "task": "t"}
    Q, K, V = [t.to(dtype).cuda().contiguous() for t in synthetic.qkv(seed, B, H, L, d, n=3)]
    mod = BlockSparseAttention(cfg, dtype=dtype, engine=_lib.ENGINE_SIMT)
    m = torch.as_tensor(mat).cuda()
    O_ref, P_ref = mod(Q, K, V, None, m)
    pat = pattern_from_mask(m, bs)
    n = B * H * pat.nnzb * bs * bs
    P = torch.zeros(n, dtype=dtype, device="cuda")
    O = torch.zeros_like(Q)
    args = (ptr(Q), ptr(K), ptr(V), None, ptr(P), ptr(O), ptr(pat.row_ptr), ptr(pat.col_idx), ptr(pat.blk_row),
            d, L, B * H, bs, pat.nnzb, _lib.F32 if dtype == torch.float32 else _lib.BF16, _lib.current_stream_ptr())
    check(lib.spion_attn_forward_static(*args), "spion_attn_forward_static")
    torch.cuda.synchronize()
    # What the entry point is for: it allocates nothing.  Checked on a repeat of the same call, so that
    # the one-off costs of a first use (the CUDA runtime loading the kernels' code and the library's
    # built-in array onto the device) are not mistaken for an allocation by the call.
    free_before = torch.cuda.mem_get_info()[0]
    check(lib.spion_attn_forward_static(*args), "spion_attn_forward_static (repeat)")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    return P, O, P_ref, O_ref


def test_static_forward_matches_ordinary_forward_twice():
    from spion_b200 import _lib
    assert _lib.lib.spion_static_scratch_capacity() == 16 * 1024 * 1024
    B, H, L, d, bs = 2, 2, 256, 64, 64
    mat1 = synthetic.band_random_mask(1, L // bs, 0.5)
    mat2 = synthetic.band_random_mask(2, L // bs, 0.3)      # fewer blocks: stale values stay behind it
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-6)):
        for seed, mat in ((101, mat1), (202, mat2)):
            P, O, P_ref, O_ref = _run_pair(dtype, seed, B, H, L, d, bs, mat)
            assert float((P.float() - P_ref.float()).abs().max()) <= tol
            assert float((O.float() - O_ref.float()).abs().max()) <= tol


def test_static_forward_rejects_oversize_and_bad_arguments():
    from spion_b200 import _lib
    lib = _lib.lib
    dummy = _lib.c_void_p(256)
    args = [dummy, dummy, dummy, None, dummy, dummy, dummy, dummy, dummy]
    # 64 (b,h) matrices x 205 blocks x 64^2 = 53.7 M values > 16 Mi: refused before any launch
    assert lib.spion_attn_forward_static(*args, 64, 4096, 64, 64, 205, _lib.BF16, None) == -2
    assert lib.spion_attn_forward_static(*args, 64, 100, 4, 64, 1, _lib.BF16, None) == -2     # ragged length
    assert lib.spion_attn_forward_static(None, *args[1:], 64, 128, 4, 64, 1, _lib.BF16, None) == -1
    assert lib.spion_attn_forward_static(*args, 64, 128, 4, 64, 5, _lib.BF16, None) == -2       # nnzb > nb*nb
