"""Multi-head attention module: the host-side mirror of the reference's ``models/attention.py``.

``Attention(config, inference=False)`` has the reference's parameters (``W_q``, ``W_k``, ``W_v``,
``ff``), ``forward(X, mask, mat=None)`` -> ``(out, attn)``, and ``reconstruct_for_blocksparse
(config)`` which switches the layer from the dense warm-up path to the sparse path
(models/attention.py:105-129).  The four ``_*_compile_module`` loaders bind the same symbol
names with the same ``argtypes`` as the reference's (models/attention.py:141-191), but load the
shims built next to ``libspion_b200.so`` instead of ``./models/*.so``.

Config keys read: head_dim, num_head, max_seq_len, batch_size, block_size, task, transformer_dim
(the reference's), plus optional ``native`` (bool: use the block-tile kernels) and ``dtype``
("fp32" | "bf16", native only).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int

import torch
import torch.nn as nn

from . import _lib

# tasks whose inputs carry padding and therefore use the key-padding variants (models/attention.py:11)
mask_task = ['lra-listops', 'lra-text', 'lra-news', 'lra-yelp', 'lra-text1', 'lra-news1', 'lra-yelp1',
             'lra-text2', 'lra-news2', 'lra-yelp2', 'lra-retrieval']

_P = ctypes.c_void_p


def _load_shim(name, n_init, n_fwd, n_bwd, trailing_int):
    path = os.path.join(_lib.LIB_DIR, name)
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run python -m spion_b200.build (there is no fallback)")
    cpp = ctypes.CDLL(path)
    cpp.init.argtypes = [c_int] * n_init
    cpp.init.restype = _P
    cpp.attn_forward.argtypes = [_P] * n_fwd + ([c_int] if trailing_int else [])
    cpp.attn_backward.argtypes = [_P] * n_bwd + ([c_int] if trailing_int else [])
    cpp.destroy.argtypes = [_P]
    return cpp


class Attention(nn.Module):
    def __init__(self, config, inference=False):
        super().__init__()
        self.inference = inference
        self.dim = config["transformer_dim"]
        self.head_dim = config["head_dim"]
        self.num_head = config["num_head"]
        self.seq_len = config["max_seq_len"]
        self.block_size = config["block_size"]
        self.num_blocks = int(self.seq_len / self.block_size)
        self.native = bool(config.get("native", False))
        self.native_dtype = torch.bfloat16 if config.get("dtype", "fp32") == "bf16" else torch.float32
        self.with_keypad = config["task"] in mask_task

        # same parameters and forward arithmetic as nn.Linear (models/attention.py:55-57); on the native path the
        # bias gradient of the backward is summed by the library's column-sum kernel
        Linear = nn.Linear
        if config.get("native") and config.get("fused_bias_grad", True):
            from .layernorm import BiasGradLinear as Linear
        self.W_q = Linear(self.dim, self.num_head * self.head_dim)
        self.W_k = Linear(self.dim, self.num_head * self.head_dim)
        self.W_v = Linear(self.dim, self.num_head * self.head_dim)

        if not inference and self.native:
            from .native import DenseViaBlocks
            self.attn = DenseViaBlocks(config, dtype=self.native_dtype, keypad=self.with_keypad)
        elif not inference:
            num_batches = config["num_head"] * config["batch_size"]
            if self.with_keypad:
                attn_cpp = Attention._cuda_mask_compile_module()
                from .attention_cuda_mask import CUDAMaskAttention as Dense
            else:
                attn_cpp = Attention._cuda_compile_module()
                from .attention_cuda import CUDAAttention as Dense
            attn_handle = attn_cpp.init(config["head_dim"], config["max_seq_len"], num_batches)
            if not attn_handle:
                raise _lib.SpionError("init() of the dense attention library returned NULL")
            self.attn = Dense(config, attn_cpp, attn_handle)

        self.ff = Linear(self.num_head * self.head_dim, self.dim)

    def forward(self, X, mask, mat=None):
        Q = self.split_heads(self.W_q(X))
        K = self.split_heads(self.W_k(X))
        V = self.split_heads(self.W_v(X))
        with torch.autocast(device_type="cuda", enabled=False):
            if mat is None and self.native:
                attn_out, attn = self.attn(Q, K, V, mask.float())
                attn_out = attn_out.to(X.dtype)
            elif mat is None:
                attn_out, attn = self.attn(Q.float(), K.float(), V.float(), mask.float())
            elif self.native:
                attn_out, attn = self.block_attn(Q, K, V, mask.float(), mat)
                attn_out = attn_out.to(X.dtype)
            else:
                attn_out, attn = self.block_attn(Q.float(), K.float(), V.float(), mask.float(), mat)
        attn_out = self.combine_heads(attn_out)
        out = self.ff(attn_out)
        return out, attn

    def reconstruct_for_blocksparse(self, config):
        num_batches = int(config["num_head"] * config["batch_size"])
        model_dev = next(self.parameters()).device
        if self.native:
            from .native import BlockSparseAttention
            # the layer above ignores the probabilities of the sparse phase (models/model_transformer.py:137 reads
            # them in the dense phase only): none are stored
            self.block_attn = BlockSparseAttention(config, dtype=self.native_dtype, keypad=self.with_keypad,
                                                   device=model_dev, return_probs=False)
            return
        if self.with_keypad:
            block_attn_cpp = Attention._blockcuda_mask_compile_module()
            from .attention_blockcuda_mask import CUDABlockMaskAttention as Sparse
        else:
            block_attn_cpp = Attention._blockcuda_compile_module()
            from .attention_blockcuda import CUDABlockAttention as Sparse
        with torch.cuda.device(model_dev):
            handle = block_attn_cpp.init(config["head_dim"], config["max_seq_len"], num_batches, config["block_size"])
        if not handle:
            raise _lib.SpionError("init() of the block attention library returned NULL (is max_seq_len a multiple "
                                  "of block_size?)")
        self.block_attn = Sparse(config, block_attn_cpp, handle)
        self.block_attn.to(model_dev)

    def combine_heads(self, X):
        X = X.transpose(1, 2)
        return X.reshape(X.size(0), X.size(1), self.num_head * self.head_dim)

    def split_heads(self, X):
        X = X.reshape(X.size(0), X.size(1), self.num_head, self.head_dim)
        return X.transpose(1, 2)

    # ---- loaders: same symbols and argtypes as models/attention.py:141-191 -------------------
    @staticmethod
    def _cuda_compile_module():
        return _load_shim("attn.so", 3, 6, 12, False)

    @staticmethod
    def _blockcuda_compile_module():
        return _load_shim("block_attn.so", 4, 9, 14, True)

    @staticmethod
    def _cuda_mask_compile_module():
        return _load_shim("attn_mask.so", 3, 7, 12, False)

    @staticmethod
    def _blockcuda_mask_compile_module():
        return _load_shim("block_attn_mask.so", 4, 10, 14, True)
