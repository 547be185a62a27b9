"""Pattern discovery on the GPU: the host-side mirror of the reference driver's pattern block.

The reference does this inline in its training loop (main_conv_ff.py:249-306): copy each
layer's mean attention map to the CPU, ``F.conv2d`` with a 31x31 diagonal filter,
``F.avg_pool2d``, ``torch.quantile``, 2*nb recursive ``flood_fill`` walkers, force the
diagonal, stack.  Here one C call per layer (``spion_discover_pattern``) does all of it on
the device and also emits the block CSR/CSC the attention kernels use.
"""
from __future__ import annotations

import pickle
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, lib, ptr

CONV_KINDS = {"diag": _lib.CONV_DIAG, "box": _lib.CONV_BOX}


@dataclass
class BlockPattern:
    """One layer's block mask and its sparse structure (all tensors on the device)."""
    block_size: int
    nb: int
    nnzb: int
    mat: torch.Tensor        # [nb, nb] uint8
    pooled: torch.Tensor     # [nb, nb] fp32 (conv + average pool of the map)
    thresh: torch.Tensor     # [1] fp32
    row_ptr: torch.Tensor    # [nb+1] int32
    col_idx: torch.Tensor    # [nnzb] int32
    blk_row: torch.Tensor    # [nnzb] int32
    col_ptr: torch.Tensor    # [nb+1] int32
    row_idx: torch.Tensor    # [nnzb] int32
    csc_pos: torch.Tensor    # [nnzb] int32

    @property
    def density(self) -> float:
        return self.nnzb / float(self.nb * self.nb)

    def float_mat(self) -> torch.Tensor:
        """The 0/1 fp32 [nb, nb] tensor the reference passes around (main_conv_ff.py:276)."""
        return self.mat.to(torch.float32)

    def element_csr(self, repeat: int = 1):
        """sum_mat [L], Offsets [L+1], Columns [repeat*nnz] (int32) and nnz, as
        models/attention_blockcuda.py:31-43 builds them on every forward call."""
        return expand_csr(self.row_ptr, self.col_idx, self.nb, self.block_size, self.nnzb, repeat)


def _alloc_structure(nb: int, device):
    i32 = dict(dtype=torch.int32, device=device)
    cap = nb * nb
    return dict(
        mat=torch.empty(nb, nb, dtype=torch.uint8, device=device),
        nnzb_dev=torch.zeros(1, **i32),
        row_ptr=torch.empty(nb + 1, **i32), col_idx=torch.empty(cap, **i32), blk_row=torch.empty(cap, **i32),
        col_ptr=torch.empty(nb + 1, **i32), row_idx=torch.empty(cap, **i32), csc_pos=torch.empty(cap, **i32),
        work=torch.empty(cap, **i32),
    )


def discover_pattern(A: torch.Tensor, block_size: int, threshold: float, conv: str = "diag", F: int = 31,
                     select: str = "paths") -> BlockPattern:
    """SPION-CF (select='paths', ``threshold`` = quantile q, main_conv_ff.py:268), SPION-C
    (select='topk', ``threshold`` = density, main_conv.py:247) or SPION-F (F=1, main_ff.py:255).

    ``A`` is the [L, L] fp32 mean attention map on the GPU.
    """
    if not A.is_cuda:
        raise ValueError("discover_pattern needs the attention map on the GPU (there is no CPU path)")
    A = A.detach().to(torch.float32).contiguous()
    L = A.shape[0]
    if A.dim() != 2 or A.shape[1] != L or L % block_size != 0:
        raise ValueError("A must be [L, L] with L a multiple of block_size")
    nb = L // block_size
    s = _alloc_structure(nb, A.device)
    pooled = torch.empty(nb, nb, dtype=torch.float32, device=A.device)
    thresh = torch.zeros(1, dtype=torch.float32, device=A.device)
    host_n = _lib.ctypes.c_int32(0)
    with torch.cuda.device(A.device):
        check(lib.spion_discover_pattern(
            ptr(A), L, block_size, CONV_KINDS[conv], F,
            _lib.SELECT_PATHS if select == "paths" else _lib.SELECT_TOPK, float(threshold),
            ptr(s["mat"]), ptr(pooled), ptr(thresh), ptr(s["nnzb_dev"]),
            ptr(s["row_ptr"]), ptr(s["col_idx"]), ptr(s["blk_row"]),
            ptr(s["col_ptr"]), ptr(s["row_idx"]), ptr(s["csc_pos"]), ptr(s["work"]),
            _lib.ctypes.cast(_lib.ctypes.byref(host_n), _lib.c_void_p), _lib.current_stream_ptr()),
            "spion_discover_pattern")
    n = int(host_n.value)
    return BlockPattern(block_size, nb, n, s["mat"], pooled, thresh, s["row_ptr"], s["col_idx"][:n], s["blk_row"][:n],
                        s["col_ptr"], s["row_idx"][:n], s["csc_pos"][:n])


def pattern_from_mask(mat: torch.Tensor, block_size: int) -> BlockPattern:
    """Structure of a given mask (any dtype, non-zero = selected), e.g. one loaded from the
    reference's pickle (main_inference.py:164-166)."""
    if not mat.is_cuda:
        raise ValueError("mask must be on the GPU")
    nb = mat.shape[0]
    s = _alloc_structure(nb, mat.device)
    s["mat"].copy_((mat != 0).to(torch.uint8))
    host_n = _lib.ctypes.c_int32(0)
    with torch.cuda.device(mat.device):
        check(lib.spion_build_structure(
            ptr(s["mat"]), nb, ptr(s["nnzb_dev"]), ptr(s["row_ptr"]), ptr(s["col_idx"]), ptr(s["blk_row"]),
            ptr(s["col_ptr"]), ptr(s["row_idx"]), ptr(s["csc_pos"]), ptr(s["work"]),
            _lib.ctypes.cast(_lib.ctypes.byref(host_n), _lib.c_void_p), _lib.current_stream_ptr()),
            "spion_build_structure")
    n = int(host_n.value)
    z = torch.zeros(0, device=mat.device)
    return BlockPattern(block_size, nb, n, s["mat"], z, z, s["row_ptr"], s["col_idx"][:n], s["blk_row"][:n],
                        s["col_ptr"], s["row_idx"][:n], s["csc_pos"][:n])


def expand_csr(row_ptr, col_idx, nb: int, block_size: int, nnzb: int, repeat: int = 1):
    dev = row_ptr.device
    L = nb * block_size
    nnz = nnzb * block_size * block_size
    sum_mat = torch.empty(L, dtype=torch.int32, device=dev)
    offsets = torch.empty(L + 1, dtype=torch.int32, device=dev)
    columns = torch.empty(max(1, repeat * nnz), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        check(lib.spion_expand_csr(ptr(row_ptr), ptr(col_idx), nb, block_size, nnzb, repeat, ptr(sum_mat),
                                   ptr(offsets), ptr(columns), _lib.current_stream_ptr()), "spion_expand_csr")
    return sum_mat, offsets, columns[:repeat * nnz], nnz


def mean_attention_map(attn: torch.Tensor, transposed_storage: bool = False) -> torch.Tensor:
    """A = mean over batch then heads of attn [B, H, L, L] (models/model_transformer.py:137).
    ``transposed_storage``: the memory holds attn[b,h,j,i] (what the dense forward writes)."""
    B, H, L, _ = attn.shape
    if not attn.is_contiguous():
        raise ValueError("attn must be contiguous in memory; pass transposed_storage for the S^T layout")
    A = torch.empty(L, L, dtype=torch.float32, device=attn.device)
    with torch.cuda.device(attn.device):
        check(lib.spion_mean_attention_map(ptr(attn), B, H, L, int(transposed_storage), ptr(A),
                                           _lib.current_stream_ptr()), "spion_mean_attention_map")
    return A


def discover_layers(attn_lst, model_config, conv: str = "diag", F: int = 31, select: str = "paths"):
    """The reference driver's loop over layers (main_conv_ff.py:254-299).

    attn_lst: per layer, the [L, L] mean attention map.  Returns (mat_lst, patterns) where
    mat_lst is the [4, layers, nb, nb] fp32 tensor the reference stacks at :298-299 (four
    copies, one per DataParallel replica) and patterns the per-layer ``BlockPattern``s.
    """
    bs = model_config["block_size"]
    L = model_config["max_seq_len"]
    key = model_config["threshold"] if select == "paths" else model_config["density"]
    patterns = [discover_pattern(a[:L], bs, key, conv, F, select) for a in attn_lst]
    mats = torch.stack([p.float_mat() for p in patterns], 0)
    return torch.stack([mats, mats, mats, mats], 0), patterns


def save_mask_pickle(mat_lst: torch.Tensor, path: str) -> None:
    """Same on-disk form as main_conv_ff.py:302-306 (pickle of the stacked tensor)."""
    with open(path, "wb") as f:
        pickle.dump(mat_lst, f, pickle.HIGHEST_PROTOCOL)


def load_mask_pickle(path: str) -> torch.Tensor:
    with open(path, "rb") as f:
        return pickle.load(f)
