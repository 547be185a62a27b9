"""Generate the golden fixtures in this folder by running the reference's own Python.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py /path/to/SPION [--large]

(``--large`` writes only pattern_reference_large.npz: the two largest block counts, minutes of CPU time.)

It imports ``main_conv_ff.flood_fill`` and ``models.attention.SoftmaxAttention`` from the
reference and executes the reference driver's pattern lines (main_conv_ff.py:255-279)
and CSR lines (models/attention_blockcuda.py:31-43) on CPU tensors.  Inputs are seeded
(``spion_b200.synthetic``); each fixture stores the seed, a SHA-256 of the input map and
the reference's outputs, so the tests can regenerate the input and compare.
Nothing here is needed at test time; the .npz files are.
"""
import hashlib
import os
import sys

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from spion_b200 import synthetic  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def reference_pattern(flood_fill, data: torch.Tensor, block_size: int, q: float, Fk: int, kind: str):
    """main_conv_ff.py:255-279 with the filter as a parameter and ff_mat on the CPU."""
    L = data.shape[0]
    num_blocks = int(L / block_size)
    if Fk > 1:
        if kind == "diag":
            kernel = np.zeros((Fk, Fk))
            np.fill_diagonal(kernel, 1)
        else:
            kernel = np.full((Fk, Fk), 1.0 / (Fk * Fk))
        kernel = np.repeat(kernel[np.newaxis, :, :], 1, axis=0)
        kernel = torch.Tensor(kernel)
        kernel = torch.unsqueeze(kernel, 0)
        out = F.conv2d(torch.unsqueeze(data, 0), kernel, stride=1, padding='same')
    else:
        out = torch.unsqueeze(data, 0)                      # main_ff.py:255
    out = F.avg_pool2d(out, (block_size, block_size))
    out = out[0]
    tmp = torch.zeros((num_blocks + 1, num_blocks + 1), dtype=torch.float32)
    tmp[:-1, :-1] = out
    thresh = torch.quantile(out, q)
    ff_mat = torch.zeros((num_blocks, num_blocks), dtype=torch.float32)
    for k in range(int(out.shape[0])):
        flood_fill(tmp, 0, k, ff_mat, thresh)
    for k in range(int(out.shape[1])):
        flood_fill(tmp, k, 0, ff_mat, thresh)
    mat = torch.where(ff_mat > 0, 1.0, 0.0)
    for i in range(num_blocks):
        mat[i, i] = 1
    return mat.numpy().astype(np.uint8), np.float32(thresh.item()), out.numpy().astype(np.float32)


def reference_topk(data, block_size, density, Fk=31):
    """main_conv.py:237-255 on the CPU."""
    L = data.shape[0]
    num_blocks = int(L / block_size)
    kernel = np.zeros((Fk, Fk))
    np.fill_diagonal(kernel, 1)
    kernel = torch.Tensor(kernel)[None, None]
    out = F.conv2d(torch.unsqueeze(data, 0), kernel, stride=1, padding='same')
    out = F.avg_pool2d(out, (block_size, block_size))[0]
    attn_pattern = out.reshape(-1)
    topk = torch.topk(attn_pattern, int(attn_pattern.shape[0] * density - num_blocks))[1]
    mat = torch.zeros((num_blocks * num_blocks), dtype=torch.float32)
    mat[topk] = 1
    mat = mat.reshape(num_blocks, num_blocks)
    for i in range(num_blocks):
        mat[i, i] = 1
    return mat.numpy().astype(np.uint8)


def reference_csr(mat_np, block_size, num_batches):
    """models/attention_blockcuda.py:31-43 on CPU tensors."""
    mat = torch.as_tensor(mat_np.astype(np.float32))
    seq_len = mat.shape[0] * block_size
    upsample = nn.Upsample(scale_factor=block_size, mode='nearest')
    sum_mat = torch.sum(mat, dim=1, dtype=torch.int32) * block_size
    sum_mat = sum_mat.repeat(block_size, 1)
    sum_mat = sum_mat.transpose(1, 0).flatten()
    Offsets = torch.zeros((seq_len + 1), dtype=torch.int32)
    cum_sum_mat = torch.cumsum(sum_mat, dim=0)
    Offsets[1:] = torch.add(Offsets[:-1], cum_sum_mat)
    nnz = Offsets[-1]
    dense_matrix = upsample(mat.unsqueeze(0).unsqueeze(0))
    col_indices = dense_matrix[0][0].nonzero()[:, 1]
    Columns = col_indices.repeat(num_batches).to(torch.int32)
    return sum_mat.numpy().astype(np.int32), Offsets.numpy(), Columns.numpy(), int(nnz)


# (name, map kind, seed, L, bs, q, F, conv kind)
PATTERN_CASES = [
    ("qk_L256_bs32_q75_diag31", "qk", 11, 256, 32, 0.75, 31, "diag"),
    ("qk_L512_bs32_q90_diag31", "qk", 12, 512, 32, 0.90, 31, "diag"),
    ("qk_L1024_bs32_q75_diag31", "qk", 1, 1024, 32, 0.75, 31, "diag"),      # benchmark config 1 shape
    ("qk_L1024_bs32_q75_box3", "qk", 1, 1024, 32, 0.75, 3, "box"),          # config 1 wording (3x3 mean)
    ("qk_L1024_bs64_q85_diag31", "qk", 13, 1024, 64, 0.85, 31, "diag"),
    ("st_L512_bs32_q85_diag31", "st", 21, 512, 32, 0.85, 31, "diag"),
    ("st_L1024_bs32_q96_diag31", "st", 22, 1024, 32, 0.96, 31, "diag"),     # image task threshold
    ("st_L1024_bs32_q90_nofilter", "st", 23, 1024, 32, 0.90, 1, "diag"),    # SPION-F
    ("st_L2048_bs64_q92_diag31", "st", 24, 2048, 64, 0.92, 31, "diag"),
    ("qk_L4096_bs64_q96_diag31", "qk", 3, 4096, 64, 0.96, 31, "diag"),      # config 3/5 shape
    ("st_L4096_bs64_q95_diag31", "st", 25, 4096, 64, 0.95, 31, "diag"),
    ("st_L4096_bs32_q95_diag31", "st", 26, 4096, 32, 0.95, 31, "diag"),     # nb = 128
    ("st_L2048_bs64_q99_diag31", "st", 27, 2048, 64, 0.99, 31, "diag"),     # text task threshold
]


# largest block counts of the kernel sweep (nb = 256, 512); stored without the pooled map (mask, threshold, CSR hash)
LARGE_CASES = [
    ("st_L8192_bs32_q97_diag31", "st", 28, 8192, 32, 0.97, 31, "diag"),     # nb = 256
    ("st_L16384_bs32_q99_diag31", "st", 29, 16384, 32, 0.99, 31, "diag"),   # nb = 512
]


def make_map(kind, seed, L):
    if kind == "qk":
        Q, K = synthetic.qkv(seed, 2, 2, L, 32, n=2)
        return synthetic.mean_attention_map(Q, K)
    return synthetic.structured_map(seed, L)


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.setrecursionlimit(10000)
    cwd = os.getcwd()
    os.chdir(ref_root)
    import main_conv_ff                                    # the reference driver module
    from models.attention import SoftmaxAttention          # the reference dense oracle
    os.chdir(cwd)

    if "--large" in sys.argv:
        big = {}
        for name, kind, seed, L, bs, q, Fk, ck in LARGE_CASES:
            A = make_map(kind, seed, L)
            mat, thresh, _ = reference_pattern(main_conv_ff.flood_fill, A, bs, q, Fk, ck)
            sm, off, col, nnz = reference_csr(mat, bs, 1)
            big[name + "/meta"] = np.array([seed, L, bs, Fk, 0 if ck == "diag" else 1, 0 if kind == "qk" else 1], np.int64)
            big[name + "/q"] = np.float64(q)
            big[name + "/sha"] = np.frombuffer(bytes.fromhex(sha(A.numpy())), dtype=np.uint8)
            big[name + "/mat"] = np.packbits(mat)
            big[name + "/thresh"] = thresh
            big[name + "/csr_sha"] = np.frombuffer(bytes.fromhex(sha(np.concatenate([sm, off, col]))), dtype=np.uint8)
            big[name + "/nnz"] = np.int64(nnz)
            print(name, "nnzb", int(mat.sum()), "density %.4f" % (mat.mean()), "thresh", thresh)
        np.savez_compressed(os.path.join(HERE, "pattern_reference_large.npz"), **big)
        return

    pat = {}
    for name, kind, seed, L, bs, q, Fk, ck in PATTERN_CASES:
        A = make_map(kind, seed, L)
        mat, thresh, pooled = reference_pattern(main_conv_ff.flood_fill, A, bs, q, Fk, ck)
        sm, off, col, nnz = reference_csr(mat, bs, 1)
        pat[name + "/meta"] = np.array([seed, L, bs, Fk, 0 if ck == "diag" else 1, 0 if kind == "qk" else 1], np.int64)
        pat[name + "/q"] = np.float64(q)
        pat[name + "/sha"] = np.frombuffer(bytes.fromhex(sha(A.numpy())), dtype=np.uint8)
        pat[name + "/mat"] = np.packbits(mat)
        pat[name + "/thresh"] = thresh
        pat[name + "/pooled"] = pooled
        pat[name + "/csr_sha"] = np.frombuffer(bytes.fromhex(sha(np.concatenate([sm, off, col]))), dtype=np.uint8)
        pat[name + "/nnz"] = np.int64(nnz)
        print(name, "nnzb", int(mat.sum()), "density %.3f" % (mat.mean()), "thresh", thresh)
    np.savez_compressed(os.path.join(HERE, "pattern_reference.npz"), **pat)

    # small CSR vectors stored in full
    csr = {}
    for name, nb, bs, dens, seed in [("nb4_bs32", 4, 32, 0.4, 5), ("nb8_bs32", 8, 32, 0.3, 6), ("nb8_bs64", 8, 64, 0.2, 7)]:
        mat = synthetic.band_random_mask(seed, nb, dens)
        sm, off, col, nnz = reference_csr(mat, bs, 2)
        csr[name + "/mat"] = mat
        csr[name + "/bs"] = np.int64(bs)
        csr[name + "/sum_mat"] = sm
        csr[name + "/offsets"] = off
        csr[name + "/columns"] = col
        csr[name + "/nnz"] = np.int64(nnz)
    np.savez_compressed(os.path.join(HERE, "csr_reference.npz"), **csr)

    # SPION-C top-k masks
    tk = {}
    for name, seed, L, bs, dens in [("st_L512_bs32_d10", 31, 512, 32, 0.10), ("st_L1024_bs32_d04", 32, 1024, 32, 0.04 + 1.0 / 32)]:
        A = synthetic.structured_map(seed, L)
        tk[name + "/meta"] = np.array([seed, L, bs], np.int64)
        tk[name + "/density"] = np.float64(dens)
        tk[name + "/mat"] = np.packbits(reference_topk(A, bs, dens))
    np.savez_compressed(os.path.join(HERE, "topk_reference.npz"), **tk)

    # dense softmax attention through the reference's SoftmaxAttention
    att = {}
    for name, seed, B, H, L, d in [("B2H2L64d32", 41, 2, 2, 64, 32), ("B1H2L128d64", 42, 1, 2, 128, 64)]:
        Q, K, V = synthetic.qkv(seed, B, H, L, d, n=3)
        kp = synthetic.key_padding(seed, B, L)
        mod = SoftmaxAttention({"attention_dropout": 0.0, "head_dim": d}, False).eval()
        out, attn = mod(Q, K, V, kp)
        att[name + "/meta"] = np.array([seed, B, H, L, d], np.int64)
        att[name + "/out"] = out.numpy()
        att[name + "/attn_rowsum"] = attn.sum(-1).numpy()
        att[name + "/attn_sha"] = np.frombuffer(bytes.fromhex(sha(attn.numpy())), dtype=np.uint8)
        att[name + "/attn_sample"] = attn[:, :, ::7, ::5].numpy()
    np.savez_compressed(os.path.join(HERE, "dense_attention_reference.npz"), **att)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else
         os.environ.get("SPION_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference")))
