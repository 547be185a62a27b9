"""Native (block-tile) sparse attention module: the B200-first entry point.

Same call shape as the reference's sparse modules -- ``forward(query, key, value, mask, mat)``
-> ``(out, attn)`` with ``[B, H, L, d]`` tensors -- but without the reference's per-call costs:

* fp32 *or* bf16 elements (the reference forces fp32, models/attention.py:88-92);
* no transposed copies of K (forward) and V (backward) (models/attention_blockcuda.py:48,80);
* block CSR/CSC fixed once per layer (``set_mask``), not rebuilt per call (:26-43);
* P is kept as ``[BH, nnzb, bs, bs]`` tiles, which is what TMA and the tensor cores want;
* on the tensor-core engine, head-split *views* of the ``[B, L, H*d]`` projections (what
  ``split_heads`` returns, models/attention.py:131-139) are read in place and the output is written
  in the same form, so neither the head split nor ``combine_heads`` copies anything.

``attn`` is returned in that tile layout (use ``to_reference_order`` to compare with the
reference's element-CSR order).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._lib import check, lib, ptr

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


class ProbsHandle:
    """What a fused forward that stores no probabilities hands back in place of them: the operands and the
    per-row log-sum-exp from which any part of P can be rebuilt (``mean_attention_map`` does, for the
    warm-up phase).  Valid until the module's next forward."""

    def __init__(self, q, k, lse, pen, heads):
        self.q, self.k, self.lse, self.pen, self.heads = q, k, lse, pen, heads


class BlockSparseAttention(nn.Module):
    def __init__(self, config, dtype=torch.float32, keypad: bool = False, engine: int = _lib.ENGINE_AUTO,
                 device=None, fused=None, return_probs: bool = True, recompute=None, block32: str = "auto"):
        super().__init__()
        self.d = config["head_dim"]
        self.H = config["num_head"]
        self.L = config["max_seq_len"]
        self.B = config["batch_size"]
        self.bs = config["block_size"]
        self.BH = self.B * self.H
        self.dtype = dtype
        self.keypad = keypad
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        kind = _lib.KIND_BLOCK_KPM if keypad else _lib.KIND_BLOCK
        h = lib.spion_create(kind, self.d, self.L, self.BH, self.bs, _DTYPES[dtype], self.device.index or 0)
        if not h:
            raise _lib.SpionError("spion_create failed (unsupported shape, or no CUDA device)")
        self.handle = _lib.c_void_p(h)
        check(lib.spion_set_engine(self.handle, engine), "spion_set_engine")
        self.engine = engine
        # 32-wide masks, bf16, head_dim 64, calls without stored probabilities: kernels on the mask's own blocks
        # ("own"), on 64-wide super-blocks ("super"), or chosen per mask by how full the gathered operands are
        check(lib.spion_set_block32_path(self.handle, {"auto": 0, "own": 1, "super": 2}[block32]), "spion_set_block32_path")
        self.needs_scratch = bool(lib.spion_needs_scratch(self.handle))
        # fused kernels (S, P, dP, dS stay on chip) where the tensor-core engine covers the shape
        can_fuse = bool(lib.spion_supports_fused(self.handle))
        if fused and not can_fuse:
            raise _lib.SpionError("fused kernels need the tcgen05 engine (bf16, block 64, head_dim 32/64)")
        self.fused = can_fuse if fused is None else bool(fused)
        # return_probs=False (fused kernels only): the forward writes O and the log-sum-exp, nothing of size
        # nnz, and ``forward`` returns a ProbsHandle instead of the [BH, nnzb, bs, bs] tiles
        self.return_probs = bool(return_probs) or not self.fused
        # recompute=True (fused kernels): the backward rebuilds P and dS on chip from the log-sum-exp and nothing
        # of size nnz exists in memory; False: the forward stores P, the backward reads it and writes dS
        # (spion_attn_backward_ex).  None: chosen per mask in set_mask -- recompute for 32-wide blocks (no tile
        # conversion passes: measured 6 - 25 % faster) and for the full mask of the warm-up phase (equal speed,
        # 2 * BH * L^2 elements less memory); stored tiles for sparse 64-wide masks (measured 10 - 15 % faster).
        self._recompute_arg = recompute
        self.recompute = self.fused and (recompute is None or bool(recompute))
        self.last = None
        self.nnzb = -1
        self._mask_key = None
        self._mask_ref = None
        self._fn = _make_function(self)

    def __del__(self):
        h = getattr(self, "handle", None)
        if h:
            lib.spion_destroy(h)
            self.handle = None

    # ------------------------------------------------------------------ pattern
    def set_mask(self, mat: torch.Tensor) -> int:
        """Fix the layer's block mask ([nb, nb], non-zero = selected).  Called once per layer at the
        dense->sparse switch, where the reference calls reconstruct_for_blocksparse."""
        m8 = (mat != 0).to(torch.uint8).contiguous().to(self.device)
        check(lib.spion_set_stream(self.handle, _lib.current_stream_ptr()))
        check(lib.spion_set_pattern(self.handle, ptr(m8)), "spion_set_pattern")
        self.nnzb = int(lib.spion_pattern_nnzb(self.handle))
        if self.fused and self._recompute_arg is None:
            nb = self.L // self.bs
            self.recompute = self.bs == 32 or self.nnzb == nb * nb
        from .pattern import pattern_from_mask
        self._pattern = pattern_from_mask(m8, self.bs)          # block CSR for the helpers above
        # The key names the tensor by address and version; the tensor itself is kept alive so that the
        # address cannot be handed to another mask while the key is in use.
        self._mask_key = (mat.data_ptr(), mat._version, tuple(mat.shape), str(mat.device))
        self._mask_ref = mat
        return self.nnzb

    @property
    def nnz(self) -> int:
        return self.nnzb * self.bs * self.bs

    def mean_attention_map(self, P_tiles) -> torch.Tensor:
        """A = mean over (b,h) of the probabilities of the last forward as an [L, L] fp32 map (zero outside the
        mask): what the encoder hands to pattern discovery (models/model_transformer.py:137), without a dense
        [B, H, L, L] tensor.  ``P_tiles`` is what ``forward`` returned beside the output: the
        [BH, nnzb, bs, bs] tiles, or a ProbsHandle, in which case the map is rebuilt from Q, K and the
        log-sum-exp and no probability was ever stored."""
        if isinstance(P_tiles, ProbsHandle):
            h = P_tiles
            A = torch.empty(self.L, self.L, dtype=torch.float32, device=h.q.device)
            check(lib.spion_set_stream(self.handle, _lib.current_stream_ptr()))
            check(lib.spion_set_head_layout(self.handle, h.heads), "spion_set_head_layout")
            check(lib.spion_mean_map_recompute(self.handle, ptr(h.q), ptr(h.k), ptr(h.lse), ptr(h.pen), ptr(A)),
                  "spion_mean_map_recompute")
            return A
        pat = self._pattern
        A = torch.empty(self.L, self.L, dtype=torch.float32, device=P_tiles.device)
        check(lib.spion_mean_map_tiles(ptr(P_tiles), _DTYPES[self.dtype], ptr(pat.blk_row), ptr(pat.col_idx), self.bs,
                                       self.nnzb, self.BH, self.L, ptr(A), _lib.current_stream_ptr()),
              "spion_mean_map_tiles")
        return A

    def launch_count(self) -> int:
        return int(lib.spion_launch_count(self.handle))

    def check_device_status(self) -> None:
        check(lib.spion_check_device_status(self.handle), "device status")

    def to_reference_order(self, P_tiles: torch.Tensor, mat: torch.Tensor) -> torch.Tensor:
        """[BH, nnzb, bs, bs] tiles -> the reference's [BH, nnz] element-CSR order."""
        nb = self.L // self.bs
        m = (mat != 0).to("cpu")
        out = []
        t = P_tiles.reshape(self.BH, self.nnzb, self.bs, self.bs)
        blk = 0
        for r in range(nb):
            n = int(m[r].sum())
            rows = t[:, blk:blk + n]                       # [BH, n, bs, bs]
            out.append(rows.permute(0, 2, 1, 3).reshape(self.BH, -1))
            blk += n
        return torch.cat(out, dim=1)

    # ------------------------------------------------------------------ call
    def _check_operands(self, query, key, value, mask):
        """The kernels take sizes from the context, not from the tensors: refuse anything else loudly
        (a short last batch would otherwise read and write past the buffers)."""
        want = (self.B, self.H, self.L, self.d)
        for name, t in (("query", query), ("key", key), ("value", value)):
            if tuple(t.shape) != want:
                raise _lib.SpionError(f"{name} has shape {tuple(t.shape)}, this module was built for {want} "
                                      "(batch_size, num_head, max_seq_len, head_dim of its config)")
            if t.device != self.device:
                raise _lib.SpionError(f"{name} is on {t.device}, the module's context is on {self.device}")
        if self.keypad:
            if mask is None or tuple(mask.shape) != (self.B, self.L):
                raise _lib.SpionError(f"key-padding mask must have shape {(self.B, self.L)}")

    def operand_form(self, t) -> int:
        """0: contiguous [B, H, L, d]; H: the head-split view of a contiguous [B, L, H, d] tensor; -1: neither."""
        if t.is_contiguous():
            return 0
        if tuple(t.stride()) == (self.L * self.H * self.d, self.d, self.H * self.d, 1):
            return self.H
        return -1

    def empty_operand(self, heads: int, device):
        """Uninitialised [B, H, L, d] tensor in the given form (see operand_form)."""
        if heads:
            return torch.empty(self.B, self.L, self.H, self.d, dtype=self.dtype, device=device).transpose(1, 2)
        return torch.empty(self.B, self.H, self.L, self.d, dtype=self.dtype, device=device)

    def forward(self, query, key, value, mask=None, mat=None):
        if mat is not None and (mat.data_ptr(), mat._version, tuple(mat.shape), str(mat.device)) != self._mask_key:
            self.set_mask(mat)
        if self.nnzb < 0:
            raise _lib.SpionError("no block mask set (call set_mask or pass mat)")
        self._check_operands(query, key, value, mask)
        pen = None
        if self.keypad:
            pen = (1e6 * (1 - mask.to(torch.float32)))[:, None, :].expand(self.B, self.H, self.L).contiguous()
        out, P = self._fn.apply(query, key, value, pen)
        if not self.return_probs:
            return out, self.last
        return out, P


class DenseViaBlocks(nn.Module):
    """Warm-up (dense) attention through the same block kernels with the full mask: the dense phase of
    the reference (models/attention_cuda.py) without fp32 up-casts, transposed copies or a
    [B, H, L, L] tensor in the reference's S^T layout.  ``forward(query, key, value, mask)`` ->
    ``(out, probs)``; ``mean_attention_map(probs)`` gives the [L, L] map for pattern discovery.  On the
    tensor-core engine ``probs`` is a ProbsHandle: no probability is written in the whole dense phase."""

    def __init__(self, config, dtype=torch.float32, keypad: bool = False, device=None, return_probs: bool = False):
        super().__init__()
        self.block = BlockSparseAttention(config, dtype=dtype, keypad=keypad, device=device, return_probs=return_probs)
        nb = config["max_seq_len"] // config["block_size"]
        self.block.set_mask(torch.ones(nb, nb, dtype=torch.uint8, device=self.block.device))

    def forward(self, query, key, value, mask=None):
        return self.block(query, key, value, mask)

    def mean_attention_map(self, P_tiles):
        return self.block.mean_attention_map(P_tiles)


def _make_function(mod: BlockSparseAttention):
    class FusedBlockAttnFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, query, key, value, pen):
            q, k, v = query.to(mod.dtype), key.to(mod.dtype), value.to(mod.dtype)
            # head-split views of [B, L, H*d] projections are read where they lie; anything else is packed
            heads = mod.H if all(mod.operand_form(t) == mod.H for t in (q, k, v)) else 0
            if not heads:
                q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
            dev = q.device
            O = mod.empty_operand(heads, dev)
            lse = torch.empty(mod.BH * mod.L, dtype=torch.float32, device=dev)
            # the probabilities are stored only for callers that want them back; the backward rebuilds its tiles
            want_p = mod.return_probs or not mod.recompute
            P = torch.empty(mod.BH * mod.nnz, dtype=mod.dtype, device=dev) if want_p else None
            check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
            check(lib.spion_set_head_layout(mod.handle, heads), "spion_set_head_layout")
            check(lib.spion_attn_forward_fused(mod.handle, ptr(q), ptr(k), ptr(v), ptr(pen), ptr(O), ptr(lse), ptr(P)),
                  "spion_attn_forward_fused")
            ctx.save_for_backward(q, k, v, O, lse)
            ctx.pen = pen
            ctx.heads = heads
            ctx.P = None if mod.recompute else P
            mod.last = ProbsHandle(q.detach(), k.detach(), lse, pen, heads)
            if P is None:
                P = torch.empty(0, dtype=mod.dtype, device=dev)
            ctx.mark_non_differentiable(P)
            # without this the engine hands the backward a zero-filled gradient of the size of the probabilities
            ctx.set_materialize_grads(False)
            return O, P

        @staticmethod
        def backward(ctx, grad_output, grad_p):
            q, k, v, O, lse = ctx.saved_tensors
            dev = q.device
            heads = ctx.heads
            go = grad_output.to(mod.dtype)
            if heads and mod.operand_form(go) != heads:
                go = go.transpose(1, 2).contiguous().transpose(1, 2)
            elif not heads:
                go = go.contiguous()
            dq, dk, dv = (mod.empty_operand(heads, dev) for _ in range(3))
            check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
            check(lib.spion_set_head_layout(mod.handle, heads), "spion_set_head_layout")
            if ctx.P is None:
                check(lib.spion_attn_backward_fused(mod.handle, ptr(q), ptr(k), ptr(v), ptr(O), ptr(go), ptr(lse),
                                                    ptr(ctx.pen), ptr(dq), ptr(dk), ptr(dv)), "spion_attn_backward_fused")
            else:
                dS = torch.empty(mod.BH * mod.nnz, dtype=mod.dtype, device=dev)
                check(lib.spion_attn_backward_ex(mod.handle, ptr(q), ptr(k), ptr(v), ptr(ctx.P), ptr(O), ptr(go), ptr(dS),
                                                 None, None, ptr(dq), ptr(dk), ptr(dv)), "spion_attn_backward_ex")
            return dq, dk, dv, None

    if mod.fused:
        return FusedBlockAttnFunction

    class NativeBlockAttnFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, query, key, value, pen):
            q = query.to(mod.dtype).contiguous()
            k = key.to(mod.dtype).contiguous()
            v = value.to(mod.dtype).contiguous()
            dev = q.device
            n = mod.BH * mod.nnz
            P = torch.empty(n, dtype=mod.dtype, device=dev)
            O = torch.empty_like(q)
            scratch = torch.empty(n, dtype=torch.float32, device=dev) if mod.needs_scratch else None
            check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
            check(lib.spion_set_head_layout(mod.handle, 0), "spion_set_head_layout")
            check(lib.spion_attn_forward_ex(mod.handle, ptr(q), ptr(k), ptr(v), ptr(pen), ptr(P), ptr(O), ptr(scratch)),
                  "spion_attn_forward_ex")
            ctx.save_for_backward(q, k, v, P, O)
            ctx.mark_non_differentiable(P)
            # without this the engine hands the backward a zero-filled gradient of the size of the probabilities
            ctx.set_materialize_grads(False)
            return O, P

        @staticmethod
        def backward(ctx, grad_output, grad_p):
            q, k, v, P, O = ctx.saved_tensors
            dev = q.device
            go = grad_output.to(mod.dtype).contiguous()
            n = mod.BH * mod.nnz
            dS = torch.empty(n, dtype=mod.dtype, device=dev)
            scratch = torch.empty(n, dtype=torch.float32, device=dev) if mod.needs_scratch else None
            dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
            check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
            check(lib.spion_attn_backward_ex(mod.handle, ptr(q), ptr(k), ptr(v), ptr(P), ptr(O), ptr(go), ptr(dS),
                                             ptr(scratch), None, ptr(dq), ptr(dk), ptr(dv)),
                  "spion_attn_backward_ex")
            return dq, dk, dv, None

    return NativeBlockAttnFunction
