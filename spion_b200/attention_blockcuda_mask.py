"""Sparse attention autograd boundary with a key-padding mask, reference layouts.

Mirror of the reference's ``models/attention_blockcuda_mask.py`` (``CUDABlockMaskAttention``):
``mask`` is the ``[B, L]`` 1/0 token mask; padded keys inside the block mask get ``-1e6`` before
the softmax (models/block_attn_mask.cu:110).  Returns ``(out, 0)`` like the reference (:62).
"""
from __future__ import annotations

import torch.nn as nn

from .attention_blockcuda import make_block_function


class CUDABlockMaskAttention(nn.Module):
    def __init__(self, config, attn_cpp, attn_handle):
        super().__init__()
        self.attn_func = make_block_function(config, attn_cpp, attn_handle, with_keypad=True)

    def forward(self, query, key, value, mask, mat):
        out, _ = self.attn_func.apply(query, key, value, mask, mat)
        return out, 0
