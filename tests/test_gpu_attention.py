"""GPU parity of the attention path against the oracle, called through the C ABI.

Tolerances (from the benchmark spec): fp32 outputs and gradients max-abs <= 1e-4; bf16 within
2e-2 relative (max-abs error over max-abs of the reference tensor), softmax accumulated in fp32.
"""
import os

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from spion_b200 import synthetic

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
FP32_TOL = 1e-4
BF16_REL = 2e-2


def cfg(B, H, L, d, bs, task="lra-image"):
    return {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
            "transformer_dim": H * d, "task": task, "attention_dropout": 0.0}


def maxabs(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def rel(a, b):
    b = b.float().cpu()
    return float((a.float().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def run_module(mod, Q, K, V, dO, *extra):
    q = Q.cuda().requires_grad_(True); k = K.cuda().requires_grad_(True); v = V.cuda().requires_grad_(True)
    out, attn = mod(q, k, v, *extra)
    out.backward(dO.cuda().to(out.dtype))
    torch.cuda.synchronize()
    return out.detach(), attn, q.grad, k.grad, v.grad


SHAPES = [  # B, H, L, d, bs, density
    (2, 2, 128, 32, 32, 0.5),
    (1, 3, 256, 64, 64, 0.4),
    (2, 1, 256, 32, 64, 0.3),
    (1, 2, 512, 64, 32, 0.1),
]


@pytest.mark.parametrize("B,H,L,d,bs,dens", SHAPES)
@pytest.mark.parametrize("kpm", [False, True])
def test_reference_layout_sparse_fp32(B, H, L, d, bs, dens, kpm):
    from spion_b200.attention import Attention
    from spion_b200.attention_blockcuda import CUDABlockAttention
    from spion_b200.attention_blockcuda_mask import CUDABlockMaskAttention
    c = cfg(B, H, L, d, bs)
    Q, K, V, dO = synthetic.qkv(7 + L + d, B, H, L, d)
    mat = synthetic.band_random_mask(L + bs, L // bs, dens)
    kp = synthetic.key_padding(3, B, L) if kpm else torch.ones(B, L)
    cpp = Attention._blockcuda_mask_compile_module() if kpm else Attention._blockcuda_compile_module()
    handle = cpp.init(d, L, B * H, bs)
    assert handle
    mod = (CUDABlockMaskAttention if kpm else CUDABlockAttention)(c, cpp, handle)
    matf = torch.as_tensor(mat, dtype=torch.float32).cuda()
    out, attn, dq, dk, dv = run_module(mod, Q, K, V, dO, kp.cuda(), matf)
    O, P, gQ, gK, gV = oatt.sparse_attention(Q, K, V, mat, bs, kp if kpm else None, dO)
    assert maxabs(out, O) <= FP32_TOL
    assert maxabs(dq, gQ) <= FP32_TOL and maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL
    if not kpm:   # the key-padding variant returns 0 instead of the probabilities (reference behaviour)
        want = oatt.csr_values_from_dense(P.numpy(), mat, bs)
        assert maxabs(attn.view(B * H, -1), torch.as_tensor(want)) <= 1e-6
    else:
        assert attn == 0
    cpp.destroy(handle)


@pytest.mark.parametrize("kpm", [False, True])
@pytest.mark.parametrize("B,H,L,d", [(2, 2, 64, 32), (1, 2, 128, 64), (1, 1, 96, 32)])
def test_reference_layout_dense_fp32(B, H, L, d, kpm):
    from spion_b200.attention import Attention
    from spion_b200.attention_cuda import CUDAAttention
    from spion_b200.attention_cuda_mask import CUDAMaskAttention
    c = cfg(B, H, L, d, 32)
    Q, K, V, dO = synthetic.qkv(70 + L, B, H, L, d)
    kp = synthetic.key_padding(4, B, L) if kpm else torch.ones(B, L)
    cpp = Attention._cuda_mask_compile_module() if kpm else Attention._cuda_compile_module()
    handle = cpp.init(d, L, B * H)
    assert handle
    mod = (CUDAMaskAttention if kpm else CUDAAttention)(c, cpp, handle)
    out, attn, dq, dk, dv = run_module(mod, Q, K, V, dO, kp.cuda())
    O, P, gQ, gK, gV = oatt.dense_attention(Q, K, V, kp if kpm else None, dO)
    assert maxabs(out, O) <= FP32_TOL and maxabs(attn, P) <= 1e-6
    assert maxabs(dq, gQ) <= FP32_TOL and maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL
    cpp.destroy(handle)


def test_dense_matches_reference_softmax_attention_fixture():
    """Outputs of the reference's own SoftmaxAttention (made by tests/golden/make_golden.py)."""
    from spion_b200.attention import Attention
    from spion_b200.attention_cuda_mask import CUDAMaskAttention
    z = np.load(os.path.join(GOLD, "dense_attention_reference.npz"))
    for cname in sorted({k.split("/")[0] for k in z.files}):
        seed, B, H, L, d = [int(x) for x in z[cname + "/meta"]]
        Q, K, V = synthetic.qkv(seed, B, H, L, d, n=3)
        kp = synthetic.key_padding(seed, B, L)
        cpp = Attention._cuda_mask_compile_module()
        handle = cpp.init(d, L, B * H)
        mod = CUDAMaskAttention(cfg(B, H, L, d, 32), cpp, handle)
        out, attn = mod(Q.cuda(), K.cuda(), V.cuda(), kp.cuda())
        assert maxabs(out, torch.as_tensor(z[cname + "/out"])) <= FP32_TOL
        assert maxabs(attn[:, :, ::7, ::5], torch.as_tensor(z[cname + "/attn_sample"])) <= 1e-6


@pytest.mark.parametrize("B,H,L,d,bs,dens", SHAPES)
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("engine", ["simt", "auto", "staged"])
def test_native_block_tiles(B, H, L, d, bs, dens, dtype, engine):
    """simt: fused fp32 kernels (bf16: one kernel per stage); staged: one kernel per stage; auto: tcgen05 for bf16."""
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    if engine == "staged" and dtype == "bf16":
        pytest.skip("same kernels as simt")
    tdt = torch.float32 if dtype == "fp32" else torch.bfloat16
    Q, K, V, dO = synthetic.qkv(11 + L + d, B, H, L, d)
    Q, K, V, dO = [t.to(tdt) for t in (Q, K, V, dO)]
    mat = synthetic.band_random_mask(L + bs + 1, L // bs, dens)
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=tdt,
                               engine={"simt": _lib.ENGINE_SIMT, "auto": _lib.ENGINE_AUTO,
                                       "staged": _lib.ENGINE_SIMT_STAGED}[engine])
    matf = torch.as_tensor(mat, dtype=torch.float32).cuda()
    out, P, dq, dk, dv = run_module(mod, Q, K, V, dO, None, matf)
    mod.check_device_status()
    O, Pd, gQ, gK, gV = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, bs, None, dO.float())
    want_tiles = torch.as_tensor(oatt.block_values_from_dense(Pd.numpy(), mat, bs))
    got_tiles = P.view(B * H, -1, bs, bs)
    if dtype == "fp32":
        assert maxabs(out, O) <= FP32_TOL and maxabs(got_tiles, want_tiles) <= 1e-6
        assert maxabs(dq, gQ) <= FP32_TOL and maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL
    else:
        assert rel(out, O) <= BF16_REL and rel(got_tiles, want_tiles) <= BF16_REL
        assert rel(dq, gQ) <= BF16_REL and rel(dk, gK) <= BF16_REL and rel(dv, gV) <= BF16_REL
    # tile layout -> reference order
    ref_order = mod.to_reference_order(P, matf)
    want = torch.as_tensor(oatt.csr_values_from_dense(Pd.numpy(), mat, bs))
    assert (rel(ref_order, want) <= BF16_REL) if dtype == "bf16" else (maxabs(ref_order, want) <= 1e-6)


def test_native_key_padding_bf16_and_fp32():
    from spion_b200.native import BlockSparseAttention
    B, H, L, d, bs = 2, 2, 256, 64, 64
    mat = synthetic.band_random_mask(5, L // bs, 0.5)
    kp = synthetic.key_padding(8, B, L)
    for tdt in (torch.float32, torch.bfloat16):
        Q, K, V, dO = [t.to(tdt) for t in synthetic.qkv(19, B, H, L, d)]
        mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=tdt, keypad=True)
        out, P, dq, dk, dv = run_module(mod, Q, K, V, dO, kp.cuda(), torch.as_tensor(mat).cuda())
        O, Pd, gQ, gK, gV = oatt.sparse_attention(Q.float(), K.float(), V.float(), mat, bs, kp, dO.float())
        if tdt == torch.float32:
            assert maxabs(out, O) <= FP32_TOL and maxabs(dq, gQ) <= FP32_TOL
            assert maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL
        else:
            assert rel(out, O) <= BF16_REL and rel(dq, gQ) <= BF16_REL
            assert rel(dk, gK) <= BF16_REL and rel(dv, gV) <= BF16_REL


def test_config1_shape_with_discovered_mask():
    """Benchmark config 1: B=8, H=2, L=1024, d=32, fp32, block 32, mask from conv + walkers."""
    from spion_b200 import pattern
    from spion_b200.attention import Attention
    from spion_b200.attention_blockcuda import CUDABlockAttention
    B, H, L, d, bs = 8, 2, 1024, 32, 32
    Q, K, V, dO = synthetic.qkv(1, B, H, L, d)
    A = synthetic.mean_attention_map(Q, K)
    pat = pattern.discover_pattern(A.cuda(), bs, 0.75)
    assert 0.10 < pat.density < 0.25
    mat = pat.mat.cpu().numpy()
    cpp = Attention._blockcuda_compile_module()
    handle = cpp.init(d, L, B * H, bs)
    mod = CUDABlockAttention(cfg(B, H, L, d, bs), cpp, handle)
    out, attn, dq, dk, dv = run_module(mod, Q, K, V, dO, torch.ones(B, L).cuda(), pat.float_mat())
    O, P, gQ, gK, gV = oatt.sparse_attention(Q, K, V, mat, bs, None, dO)
    assert maxabs(out, O) <= FP32_TOL
    assert maxabs(dq, gQ) <= FP32_TOL and maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL


def test_edge_masks_full_and_diagonal_only():
    from spion_b200.native import BlockSparseAttention
    B, H, L, d, bs = 1, 2, 256, 32, 32
    Q, K, V, dO = synthetic.qkv(23, B, H, L, d)
    for mat in (np.ones((8, 8), np.uint8), np.eye(8, dtype=np.uint8)):
        mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=torch.float32)
        out, P, dq, dk, dv = run_module(mod, Q, K, V, dO, None, torch.as_tensor(mat).cuda())
        O, Pd, gQ, gK, gV = oatt.sparse_attention(Q, K, V, mat, bs, None, dO)
        assert maxabs(out, O) <= FP32_TOL and maxabs(dq, gQ) <= FP32_TOL
        assert maxabs(dk, gK) <= FP32_TOL and maxabs(dv, gV) <= FP32_TOL
        if mat.all():   # full mask == ordinary softmax attention: rows of P sum to one
            assert abs(float(P.float().sum() / (B * H * L)) - 1.0) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_full_size_properties_L4096(dtype):
    """Benchmark sweep shape (B=8, H=8, L=4096, d=64, block 64, 5 %): size-independent checks.
       <dQ,Q> == <dK,K>, <dV,V> == <dO,O>, and sampled rows against an fp64 row oracle."""
    from spion_b200.native import BlockSparseAttention
    B, H, L, d, bs = 8, 8, 4096, 64, 64
    nb = L // bs
    mat = synthetic.band_random_mask(2024, nb, 0.05)
    Q, K, V, dO = [t.to(dtype) for t in synthetic.qkv(99, B, H, L, d)]
    mod = BlockSparseAttention(cfg(B, H, L, d, bs), dtype=dtype)
    out, P, dq, dk, dv = run_module(mod, Q, K, V, dO, None, torch.as_tensor(mat).cuda())
    mod.check_device_status()
    f = lambda t: t.double().cpu()
    a, b = float((f(dq) * f(Q)).sum()), float((f(dk) * f(K)).sum())
    c, e = float((f(dv) * f(V)).sum()), float((f(dO) * f(out)).sum())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    scale_ab = max(abs(a), abs(b), float((f(dq).abs() * f(Q).abs()).sum()) * 1e-3)
    assert abs(a - b) <= tol * scale_ab
    assert abs(c - e) <= tol * max(abs(c), abs(e), 1.0)
    rng = np.random.default_rng(0)
    for _ in range(12):
        bh, i = int(rng.integers(B * H)), int(rng.integers(L))
        bb, hh = divmod(bh, H)
        cols = np.concatenate([np.arange(cc * bs, cc * bs + bs) for cc in np.nonzero(mat[i // bs])[0]])
        s = (K[bb, hh, cols].double() @ Q[bb, hh, i].double()) / np.sqrt(d)
        p = torch.exp(s) / (torch.exp(s).sum() + (L - len(cols)))
        o = p @ V[bb, hh, cols].double()
        got = out[bb, hh, i].double().cpu()
        if dtype == torch.float32:
            assert float((got - o).abs().max()) <= FP32_TOL
        else:
            assert float((got - o).abs().max()) <= BF16_REL * float(o.abs().max()) + 1e-3


def test_errors_are_loud():
    from spion_b200 import _lib
    from spion_b200.native import BlockSparseAttention
    with pytest.raises(_lib.SpionError):
        BlockSparseAttention(cfg(1, 1, 100, 32, 32))          # ragged length
    mod = BlockSparseAttention(cfg(1, 1, 128, 32, 32))
    Q, K, V, _ = synthetic.qkv(1, 1, 1, 128, 32)
    with pytest.raises(_lib.SpionError):
        mod(Q.cuda(), K.cuda(), V.cuda())                      # no mask set
