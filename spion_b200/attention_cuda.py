"""Dense (warm-up phase) attention autograd boundary, reference layouts.

Mirror of the reference's ``models/attention_cuda.py`` (``CUDAAttention``; ``forward(query, key,
value, mask)`` -> ``(out, attn)`` with ``attn`` the full ``[B, H, L, L]`` probabilities that the
encoder averages for pattern discovery, models/model_transformer.py:137).  The native library
keeps the reference's memory conventions: Q and V are handed over as ``[BH, d, L]``, the
attention tensor is stored transposed and returned as a permuted view (:32-36).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._lib import lib, ptr
from .attention_blockcuda import _call


def make_dense_function(config, attn_cpp, attn_handle, with_keypad: bool):
    emb_dim = config["head_dim"]
    num_heads = config["num_head"]
    seq_len = config["max_seq_len"]
    batch_size = config["batch_size"]
    handle = _lib.c_void_p(attn_handle) if not isinstance(attn_handle, _lib.c_void_p) else attn_handle

    class AttnFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, query, key, value, mask):
            _lib.check_operands((batch_size, num_heads, seq_len, emb_dim), query=query, key=key, value=value)
            dev = query.device
            f32 = dict(dtype=torch.float32, device=dev)
            lib.spion_set_stream(handle, _lib.current_stream_ptr())
            qt = query.permute(0, 1, 3, 2).contiguous()
            k = key.contiguous()
            vt = value.permute(0, 1, 3, 2).contiguous()
            attn_t = torch.empty(batch_size, num_heads, seq_len, seq_len, **f32)      # attn_t[b,h,j,i] = P[i,j]
            out_t = torch.empty(batch_size, num_heads, emb_dim, seq_len, **f32)
            if with_keypad:
                pen = (1e6 * (1 - mask.to(torch.float32)))[:, None, :].expand(batch_size, num_heads, seq_len).contiguous()
                _call(attn_cpp.attn_forward, "attn_forward", handle, ptr(qt), ptr(k), ptr(vt), ptr(pen), ptr(attn_t),
                      ptr(out_t))
            else:
                _call(attn_cpp.attn_forward, "attn_forward", handle, ptr(qt), ptr(k), ptr(vt), ptr(attn_t), ptr(out_t))
            ctx.save_for_backward(qt, key, value, attn_t)
            attn = attn_t.permute(0, 1, 3, 2)
            ctx.mark_non_differentiable(attn)
            # without this the engine hands the backward a zero-filled gradient of the size of the probabilities
            ctx.set_materialize_grads(False)
            return out_t.permute(0, 1, 3, 2), attn

        @staticmethod
        def backward(ctx, grad_output, grad_weights):
            qt, key, value, attn_t = ctx.saved_tensors
            dev = qt.device
            f32 = dict(dtype=torch.float32, device=dev)
            lib.spion_set_stream(handle, _lib.current_stream_ptr())
            n = batch_size * num_heads * seq_len * seq_len
            s1 = torch.empty(n, **f32)
            s3 = torch.empty(n, **f32)
            kt = key.permute(0, 1, 3, 2).contiguous()
            v = value.contiguous()
            got = grad_output.permute(0, 1, 3, 2).contiguous()
            shape = (batch_size, num_heads, emb_dim, seq_len)
            dq, dk, dv = torch.empty(shape, **f32), torch.empty(shape, **f32), torch.empty(shape, **f32)
            # the reference passes three BH*L*L scratch buffers (:44-46); the middle one is unused here
            _call(attn_cpp.attn_backward, "attn_backward", handle, ptr(qt), ptr(kt), ptr(v), ptr(attn_t), ptr(got),
                  ptr(s1), ptr(s1), ptr(s3), ptr(dq), ptr(dk), ptr(dv))
            return dq.permute(0, 1, 3, 2), dk.permute(0, 1, 3, 2), dv.permute(0, 1, 3, 2), None

    return AttnFunction


class CUDAAttention(nn.Module):
    def __init__(self, config, attn_cpp=None, attn_handle=None):
        super().__init__()
        self.attn_func = make_dense_function(config, attn_cpp, attn_handle, with_keypad=False)

    def forward(self, query, key, value, mask):
        return self.attn_func.apply(query, key, value, mask)
