"""Sparse attention autograd boundary, reference layouts (no key-padding mask).

Mirror of the reference's ``models/attention_blockcuda.py`` (class ``CUDABlockAttention``,
``__init__(config, attn_cpp, attn_handle)``, ``forward(query, key, value, mask, mat)`` ->
``(out, attn)``): fp32 ``[B, H, L, d]`` inputs, ``attn`` = the selected probabilities in the
reference's element-CSR order ``[BH * nnz]``.  ``attn_cpp`` is a ctypes library exporting the
reference's symbols (``attn_forward`` / ``attn_backward``); ``attn_handle`` what its ``init``
returned.  Differences from the reference, all behind the same interface:

* the element CSR (``sum_mat`` / ``Offsets`` / ``Columns``) comes from one kernel
  (``spion_expand_csr``) and is cached per mask tensor instead of being rebuilt by a chain of
  torch ops with two host syncs on every call (models/attention_blockcuda.py:26-43);
* ``Columns`` is not repeated BH times (the kernels read one copy);
* a failing native call raises instead of being ignored.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._lib import SpionError, lib, ptr
from .pattern import pattern_from_mask


class _CsrCache:
    """Element CSR of the most recent mask tensor, keyed on storage pointer and version.  The keyed
    tensor is kept alive, so its address cannot be given to a different mask while the key is in use."""

    def __init__(self, block_size: int, on_new=None):
        self.block_size = block_size
        self.key = None
        self.ref = None
        self.value = None
        self.on_new = on_new          # called whenever new arrays replace the cached ones

    def get(self, mat: torch.Tensor):
        key = (mat.data_ptr(), mat._version, tuple(mat.shape), str(mat.device))
        if key != self.key:
            pat = pattern_from_mask(mat, self.block_size)
            sum_mat, offsets, columns, nnz = pat.element_csr(1)
            self.key, self.ref, self.value = key, mat, (sum_mat, offsets, columns, nnz)
            if self.on_new is not None:
                self.on_new()
        return self.value


def _call(fn, what, *args):
    rc = fn(*args)
    if rc not in (0, None):
        raise SpionError(f"{what} failed with status {rc} ({lib.spion_status_string(int(rc)).decode()})")


def make_block_function(config, attn_cpp, attn_handle, with_keypad: bool):
    emb_dim = config["head_dim"]
    num_heads = config["num_head"]
    seq_len = config["max_seq_len"]
    batch_size = config["batch_size"]
    block_size = config["block_size"]
    num_batches = batch_size * num_heads
    handle = _lib.c_void_p(attn_handle) if not isinstance(attn_handle, _lib.c_void_p) else attn_handle
    # The cache keeps the element-CSR arrays of the current mask alive and unchanged, so the library may
    # keep the block structure it derived from them; new arrays (a new mask) may reuse the old addresses,
    # so the library is told to forget what it has each time the cache is refilled.
    cache = _CsrCache(block_size, on_new=lambda: lib.spion_csr_arrays_are_stable(handle, 1))

    class BlockAttnFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, query, key, value, mask, mat):
            _lib.check_operands((batch_size, num_heads, seq_len, emb_dim), query=query, key=key, value=value)
            sum_mat, offsets, columns, nnz = cache.get(mat)
            dev = query.device
            lib.spion_set_stream(handle, _lib.current_stream_ptr())
            q = query.contiguous()
            kt = key.permute(0, 1, 3, 2).contiguous()            # [BH, d, L], as the ABI expects
            v = value.contiguous()
            attn = torch.empty(num_batches * nnz, dtype=torch.float32, device=dev)
            out = torch.empty(batch_size, num_heads, seq_len, emb_dim, dtype=torch.float32, device=dev)
            if with_keypad:
                # 1e6 on padded keys, one row per (b, h): models/attention_blockcuda_mask.py:42-43
                pen = (1e6 * (1 - mask.to(torch.float32)))[:, None, :].expand(batch_size, num_heads, seq_len).contiguous()
                _call(attn_cpp.attn_forward, "attn_forward", handle, ptr(q), ptr(kt), ptr(v), ptr(pen), ptr(attn),
                      ptr(out), ptr(offsets), ptr(columns), ptr(sum_mat), nnz)
            else:
                _call(attn_cpp.attn_forward, "attn_forward", handle, ptr(q), ptr(kt), ptr(v), ptr(attn), ptr(out),
                      ptr(offsets), ptr(columns), ptr(sum_mat), nnz)
            ctx.save_for_backward(q, key, value, attn, offsets, columns, sum_mat)
            ctx.nnz = nnz
            ctx.mark_non_differentiable(attn)
            # without this the engine hands the backward a zero-filled gradient of the size of the probabilities
            ctx.set_materialize_grads(False)
            return out, attn

        @staticmethod
        def backward(ctx, grad_output, grad_weight):
            q, key, value, attn, offsets, columns, sum_mat = ctx.saved_tensors
            nnz = ctx.nnz
            dev = q.device
            lib.spion_set_stream(handle, _lib.current_stream_ptr())
            k = key.contiguous()
            vt = value.permute(0, 1, 3, 2).contiguous()          # [BH, d, L]
            go = grad_output.contiguous()
            f32 = dict(dtype=torch.float32, device=dev)
            d_p = torch.empty(num_batches * nnz, **f32)           # the reference zero-fills this one (:84)
            d_s = torch.empty(num_batches * nnz, **f32)
            shape = (batch_size, num_heads, seq_len, emb_dim)
            dq, dk, dv = torch.empty(shape, **f32), torch.empty(shape, **f32), torch.empty(shape, **f32)
            _call(attn_cpp.attn_backward, "attn_backward", handle, ptr(q), ptr(k), ptr(vt), ptr(attn), ptr(go),
                  ptr(d_p), ptr(d_s), ptr(dq), ptr(dk), ptr(dv), ptr(offsets), ptr(columns), ptr(sum_mat), nnz)
            return dq, dk, dv, None, None

    return BlockAttnFunction


class CUDABlockAttention(nn.Module):
    def __init__(self, config, attn_cpp, attn_handle):
        super().__init__()
        self.attn_func = make_block_function(config, attn_cpp, attn_handle, with_keypad=False)

    def forward(self, query, key, value, mask, mat):
        return self.attn_func.apply(query, key, value, mask, mat)
