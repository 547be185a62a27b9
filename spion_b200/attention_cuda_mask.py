"""Dense attention with a key-padding mask, reference layouts.

Mirror of the reference's ``models/attention_cuda_mask.py`` (``CUDAMaskAttention``): padded
keys get ``-1e6`` before the softmax (models/attn_mask.cu:20).
"""
from __future__ import annotations

import torch.nn as nn

from .attention_cuda import make_dense_function


class CUDAMaskAttention(nn.Module):
    def __init__(self, config, attn_cpp=None, attn_handle=None):
        super().__init__()
        self.attn_func = make_dense_function(config, attn_cpp, attn_handle, with_keypad=True)

    def forward(self, query, key, value, mask):
        return self.attn_func.apply(query, key, value, mask)
