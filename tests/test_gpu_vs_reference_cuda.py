"""Cross-check against the reference's OWN CUDA code (cuSPARSE SDDMM/SpMM + its softmax kernels),
compiled from the reference checkout into oracle/_ref by oracle/build_ref.py.  Skipped when those
files were not built (they cannot be built where the reference checkout is absent).

The calls restate the reference's Python calling convention (models/attention_blockcuda.py:47-63,
:78-106): fp32 operands, K transposed for forward, V transposed for backward, Columns repeated
once per (b,h) matrix, dP scratch zero-filled.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from oracle import csr as ocsr
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
P = ctypes.c_void_p


def _ref_lib(name, n_init, n_fwd, n_bwd):
    path = os.path.join(REF_DIR, name)
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    lib = ctypes.CDLL(path)
    lib.init.argtypes = [ctypes.c_int] * n_init
    lib.init.restype = P
    lib.attn_forward.argtypes = [P] * n_fwd + [ctypes.c_int]
    lib.attn_backward.argtypes = [P] * n_bwd + [ctypes.c_int]
    lib.attn_forward.restype = None
    lib.attn_backward.restype = None
    return lib


def p(t):
    return P(t.data_ptr())


@pytest.mark.parametrize("B,H,L,d,bs,dens", [(2, 2, 128, 32, 32, 0.5), (1, 2, 256, 64, 64, 0.4),
                                             (8, 2, 1024, 32, 32, 0.15)])
def test_sparse_attention_matches_reference_cuda(B, H, L, d, bs, dens):
    from spion_b200.attention import Attention
    ref = _ref_lib("block_attn.so", 4, 9, 14)
    BH = B * H
    Q, K, V, dO = [t.cuda() for t in synthetic.qkv(17 + L, B, H, L, d)]
    mat = synthetic.band_random_mask(L + 3, L // bs, dens)
    sm, off, col, nnz = ocsr.element_csr(mat, bs, BH)
    sm, off, col = [torch.as_tensor(x).cuda() for x in (sm, off, col)]
    Kt = K.permute(0, 1, 3, 2).contiguous()
    Vt = V.permute(0, 1, 3, 2).contiguous()

    def run(lib, handle):
        attn = torch.empty(BH * nnz, device="cuda"); out = torch.empty(BH * L * d, device="cuda")
        lib.attn_forward(handle, p(Q), p(Kt), p(V), p(attn), p(out), p(off), p(col), p(sm), nnz)
        dP = torch.zeros(BH * nnz, device="cuda"); dS = torch.empty(BH * nnz, device="cuda")
        dQ, dK, dV = [torch.empty(BH * L * d, device="cuda") for _ in range(3)]
        lib.attn_backward(handle, p(Q), p(K), p(Vt), p(attn), p(dO.contiguous()), p(dP), p(dS), p(dQ), p(dK), p(dV),
                          p(off), p(col), p(sm), nnz)
        torch.cuda.synchronize()
        return attn, out, dQ, dK, dV

    h_ref = ref.init(d, L, BH, bs)
    r = run(ref, h_ref)
    mine = Attention._blockcuda_compile_module()
    h = mine.init(d, L, BH, bs)
    m = run(mine, h)
    names = ["attn", "out", "dQ", "dK", "dV"]
    for a, b, n in zip(m, r, names):
        err = float((a - b).abs().max())
        assert err <= 1e-4, f"{n}: max-abs {err} against the reference's CUDA path"
    # and both against the oracle
    O, Pd, gQ, gK, gV = oatt.sparse_attention(Q.cpu(), K.cpu(), V.cpu(), mat, bs, None, dO.cpu())
    want = [torch.as_tensor(oatt.csr_values_from_dense(Pd.numpy(), mat, bs)).reshape(-1), O.reshape(-1),
            gQ.reshape(-1), gK.reshape(-1), gV.reshape(-1)]
    for a, w, n in zip(r, want, names):
        err = float((a.cpu() - w).abs().max())
        assert err <= 1e-4, f"reference CUDA vs oracle, {n}: {err}"
    mine.destroy(h)


def test_sparse_keypad_matches_reference_cuda():
    from spion_b200.attention import Attention
    ref = _ref_lib("block_attn_mask.so", 4, 10, 14)
    B, H, L, d, bs = 2, 2, 256, 32, 32
    BH = B * H
    Q, K, V, dO = [t.cuda() for t in synthetic.qkv(31, B, H, L, d)]
    kp = synthetic.key_padding(5, B, L)
    pen = (1e6 * (1 - kp))[:, None, :].expand(B, H, L).contiguous().cuda()
    mat = synthetic.band_random_mask(9, L // bs, 0.4)
    sm, off, col, nnz = ocsr.element_csr(mat, bs, BH)
    sm, off, col = [torch.as_tensor(x).cuda() for x in (sm, off, col)]
    Kt = K.permute(0, 1, 3, 2).contiguous()
    outs = []
    mine = Attention._blockcuda_mask_compile_module()
    for lib in (ref, mine):
        h = lib.init(d, L, BH, bs)
        attn = torch.empty(BH * nnz, device="cuda"); out = torch.empty(BH * L * d, device="cuda")
        lib.attn_forward(h, p(Q), p(Kt), p(V), p(pen), p(attn), p(out), p(off), p(col), p(sm), nnz)
        torch.cuda.synchronize()
        outs.append((attn, out))
    assert float((outs[0][0] - outs[1][0]).abs().max()) <= 1e-5
    assert float((outs[0][1] - outs[1][1]).abs().max()) <= 1e-4
