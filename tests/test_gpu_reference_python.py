"""The drop-in claim, exercised the way the reference calls: its own, unmodified Python modules bound to
the shim libraries (when a reference checkout is present), and -- everywhere -- a restatement of what
those modules hand to the C entry points: ``Columns`` repeated once per (b,h) matrix, ``nnz`` as a
0-dim CUDA tensor that ctypes converts, a zero-filled dP scratch, flattened / permuted copies of the
operands (models/attention_blockcuda.py:26-63, :72-106; models/attention_cuda.py:17-74).

The checkout is looked for under $SPION_REFERENCE_ROOT (default ~/reference); the first test is skipped where
it does not exist.
"""
import ctypes
import importlib.util
import os
from ctypes import c_int, c_void_p

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu
REF_ROOT = os.environ.get("SPION_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))
TOL = 1e-4


def _shim(name, n_init, n_fwd, n_bwd, trailing_int):
    """Bound exactly as models/attention.py:141-191 binds ./models/<name>: same argtypes, default (int) restype
    for the calls the reference declares void."""
    from spion_b200 import _lib
    cpp = ctypes.CDLL(os.path.join(_lib.LIB_DIR, name))
    cpp.init.argtypes = [c_int] * n_init
    cpp.init.restype = c_void_p
    cpp.attn_forward.argtypes = [c_void_p] * n_fwd + ([c_int] if trailing_int else [])
    cpp.attn_backward.argtypes = [c_void_p] * n_bwd + ([c_int] if trailing_int else [])
    cpp.destroy.argtypes = [c_void_p]
    return cpp


def _config(B, H, L, d, bs):
    return {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs}


def _maxabs(a, b):
    return float((a.detach().float().cpu() - b.float().cpu()).abs().max())


def _load_reference_module(fname):
    path = os.path.join(REF_ROOT, "models", fname)
    if not REF_ROOT or not os.path.exists(path):
        pytest.skip(f"no reference checkout at {REF_ROOT}")
    spec = importlib.util.spec_from_file_location("spion_reference_" + fname[:-3], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_modules_unmodified_on_the_shims():
    """models/attention_blockcuda.py and models/attention_cuda.py, imported from the checkout as they are,
    given the shim libraries and the handle their init() returns; outputs and gradients against the oracle."""
    B, H, L, d, bs = 2, 2, 256, 32, 32
    Q, K, V, dO = synthetic.qkv(61, B, H, L, d)
    mat = synthetic.band_random_mask(3, L // bs, 0.4)

    sparse = _load_reference_module("attention_blockcuda.py")
    cpp = _shim("block_attn.so", 4, 9, 14, True)
    handle = cpp.init(d, L, B * H, bs)
    mod = sparse.CUDABlockAttention(_config(B, H, L, d, bs), cpp, handle)
    q, k, v = [t.cuda().requires_grad_(True) for t in (Q, K, V)]
    out, attn = mod(q, k, v, torch.ones(B, L).cuda(), torch.as_tensor(mat, dtype=torch.float32).cuda())
    out.backward(dO.cuda())
    torch.cuda.synchronize()
    O, P, gQ, gK, gV = oatt.sparse_attention(Q, K, V, mat, bs, None, dO)
    assert _maxabs(out, O) <= TOL
    assert _maxabs(attn.view(B * H, -1), torch.as_tensor(oatt.csr_values_from_dense(P.numpy(), mat, bs))) <= 1e-6
    assert _maxabs(q.grad, gQ) <= TOL and _maxabs(k.grad, gK) <= TOL and _maxabs(v.grad, gV) <= TOL
    cpp.destroy(handle)

    dense = _load_reference_module("attention_cuda.py")
    cpp = _shim("attn.so", 3, 6, 12, False)
    handle = cpp.init(d, L, B * H)
    mod = dense.CUDAAttention(_config(B, H, L, d, bs), cpp, handle)
    q, k, v = [t.cuda().requires_grad_(True) for t in (Q, K, V)]
    out, attn = mod(q, k, v, torch.ones(B, L).cuda())
    out.backward(dO.cuda())
    torch.cuda.synchronize()
    O, P, gQ, gK, gV = oatt.dense_attention(Q, K, V, None, dO)
    assert _maxabs(out, O) <= TOL and _maxabs(attn, P) <= 1e-6
    assert _maxabs(q.grad, gQ) <= TOL and _maxabs(k.grad, gK) <= TOL and _maxabs(v.grad, gV) <= TOL
    cpp.destroy(handle)


@pytest.mark.parametrize("B,H,L,d,bs,dens", [(2, 2, 256, 32, 32, 0.4), (1, 2, 256, 64, 64, 0.5)])
def test_sparse_entry_points_with_the_reference_calling_convention(B, H, L, d, bs, dens):
    """What models/attention_blockcuda.py builds per call, restated: the element CSR from torch ops on the
    float mask, Columns repeated B*H times, nnz = Offsets[-1] left as a 0-dim CUDA tensor (ctypes converts
    it), flattened operands with K / V permuted, dP scratch zero-filled, dS scratch uninitialised."""
    BH = B * H
    Q, K, V, dO = [t.cuda() for t in synthetic.qkv(71 + L, B, H, L, d)]
    mat_np = synthetic.band_random_mask(5 + bs, L // bs, dens)
    mat = torch.as_tensor(mat_np, dtype=torch.float32).cuda()

    per_row = (torch.sum(mat, dim=1, dtype=torch.int32) * bs).repeat(bs, 1).transpose(1, 0).flatten()
    offsets = torch.zeros(L + 1, dtype=torch.int32, device="cuda")
    offsets[1:] = torch.cumsum(per_row, dim=0)
    nnz = offsets[-1]                                              # stays a tensor, as in the reference
    dense_mask = torch.nn.Upsample(scale_factor=bs, mode="nearest")(mat[None, None])[0][0]
    columns = dense_mask.nonzero()[:, 1].repeat(BH).to(torch.int32)
    assert nnz.dim() == 0 and nnz.is_cuda

    cpp = _shim("block_attn.so", 4, 9, 14, True)
    handle = cpp.init(d, L, BH, bs)
    attn = torch.empty(BH * nnz, dtype=torch.float32, device="cuda")
    out = torch.empty(L * d * BH, dtype=torch.float32, device="cuda")
    q_flat, kt_flat, v_flat = Q.flatten(), K.permute(0, 1, 3, 2).flatten(), V.flatten()
    rc = cpp.attn_forward(handle, q_flat.data_ptr(), kt_flat.data_ptr(), v_flat.data_ptr(), attn.data_ptr(),
                          out.data_ptr(), offsets.data_ptr(), columns.data_ptr(), per_row.data_ptr(), nnz)
    assert rc == 0
    d_p = torch.zeros(int(nnz) * BH, dtype=torch.float32, device="cuda")
    d_s = torch.empty(int(nnz) * BH, dtype=torch.float32, device="cuda")
    gq, gk, gv = [torch.empty(L * d * BH, dtype=torch.float32, device="cuda") for _ in range(3)]
    vt_flat = V.permute(0, 1, 3, 2).flatten()
    rc = cpp.attn_backward(handle, q_flat.data_ptr(), K.flatten().data_ptr(), vt_flat.data_ptr(), attn.data_ptr(),
                           dO.contiguous().data_ptr(), d_p.data_ptr(), d_s.data_ptr(), gq.data_ptr(), gk.data_ptr(),
                           gv.data_ptr(), offsets.data_ptr(), columns.data_ptr(), per_row.data_ptr(), nnz)
    assert rc == 0
    torch.cuda.synchronize()
    O, P, wQ, wK, wV = oatt.sparse_attention(Q.cpu(), K.cpu(), V.cpu(), mat_np, bs, None, dO.cpu())
    shape = (B, H, L, d)
    assert _maxabs(out.view(shape), O) <= TOL
    assert _maxabs(attn.view(BH, -1), torch.as_tensor(oatt.csr_values_from_dense(P.numpy(), mat_np, bs))) <= 1e-6
    assert _maxabs(gq.view(shape), wQ) <= TOL and _maxabs(gk.view(shape), wK) <= TOL and _maxabs(gv.view(shape), wV) <= TOL
    cpp.destroy(handle)


def test_dense_entry_points_with_the_reference_calling_convention():
    """models/attention_cuda.py:17-74 restated: Q and V permuted to [B, H, d, L] copies, the attention tensor
    read back through a permuted view, three L*L scratch arrays in the backward (the first zero-filled)."""
    B, H, L, d = 2, 2, 128, 32
    BH = B * H
    Q, K, V, dO = [t.cuda() for t in synthetic.qkv(83, B, H, L, d)]
    cpp = _shim("attn.so", 3, 6, 12, False)
    handle = cpp.init(d, L, BH)
    qt = Q.permute(0, 1, 3, 2).flatten().contiguous()
    vt = V.permute(0, 1, 3, 2).flatten().contiguous()
    attn = torch.empty(B, H, L, L, dtype=torch.float32, device="cuda")
    out = torch.empty(B, H, L, d, dtype=torch.float32, device="cuda")
    assert cpp.attn_forward(handle, qt.data_ptr(), K.contiguous().data_ptr(), vt.data_ptr(), attn.data_ptr(),
                            out.data_ptr()) == 0
    s1 = torch.zeros(BH * L * L, dtype=torch.float32, device="cuda")
    s2, s3 = [torch.empty(BH * L * L, dtype=torch.float32, device="cuda") for _ in range(2)]
    gq, gk, gv = [torch.empty(B, H, L, d, dtype=torch.float32, device="cuda") for _ in range(3)]
    got = dO.permute(0, 1, 3, 2).contiguous()
    kt = K.permute(0, 1, 3, 2).flatten().contiguous()
    assert cpp.attn_backward(handle, qt.data_ptr(), kt.data_ptr(), V.flatten().data_ptr(), attn.data_ptr(), got.data_ptr(),
                             s1.data_ptr(), s2.data_ptr(), s3.data_ptr(), gq.data_ptr(), gk.data_ptr(), gv.data_ptr()) == 0
    torch.cuda.synchronize()
    O, P, wQ, wK, wV = oatt.dense_attention(Q.cpu(), K.cpu(), V.cpu(), None, dO.cpu())
    unperm = lambda t: t.view(B, H, d, L).permute(0, 1, 3, 2)
    assert _maxabs(unperm(out), O) <= TOL
    assert _maxabs(attn.view(B, H, L, L).permute(0, 1, 3, 2), P) <= 1e-6
    assert _maxabs(unperm(gq), wQ) <= TOL and _maxabs(unperm(gk), wK) <= TOL and _maxabs(unperm(gv), wV) <= TOL
    cpp.destroy(handle)
