"""Layer normalisation of the encoder layers through the library's kernels (csrc/layernorm.cu).

Same arithmetic as ``torch.nn.LayerNorm`` over the last dimension (biased variance, eps inside the root;
the reference's encoder uses that module: models/model_transformer.py).  The input is the fp32 residual
stream; the output can be bf16, which is what the linear layers that follow consume under mixed precision
(no separate cast kernels).  The backward forms dX, dweight and dbias in one pass over the rows.
"""
from __future__ import annotations

import torch
from torch import nn

from . import _lib
from ._lib import check, lib, ptr

SUPPORTED_WIDTHS = (64, 128, 256, 512)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_bf16):
        if not x.is_cuda or x.dtype != torch.float32:
            raise _lib.SpionError("FusedLayerNorm needs an fp32 CUDA tensor")
        N = x.shape[-1]
        xc = x.contiguous()
        M = xc.numel() // N
        y = torch.empty(xc.shape, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=x.device)
        mean = torch.empty(M, dtype=torch.float32, device=x.device)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        w, b = weight.float().contiguous(), bias.float().contiguous()
        with torch.cuda.device(x.device):                     # the kernels are launched on the current device
            check(lib.spion_layernorm_forward(ptr(xc), ptr(w), ptr(b), ptr(y), int(out_bf16), ptr(mean), ptr(rstd), M, N,
                                              float(eps), _lib.current_stream_ptr()), "spion_layernorm_forward")
        ctx.save_for_backward(xc, w, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w, mean, rstd = ctx.saved_tensors
        N = xc.shape[-1]
        M = xc.numel() // N
        if dy.dtype not in (torch.float32, torch.bfloat16):
            dy = dy.float()
        dy = dy.contiguous()
        dx = torch.empty_like(xc)
        dw = torch.empty(N, dtype=torch.float32, device=xc.device)
        db = torch.empty(N, dtype=torch.float32, device=xc.device)
        ws = torch.empty(int(lib.spion_layernorm_workspace_floats(N)), dtype=torch.float32, device=xc.device)
        with torch.cuda.device(xc.device):
            check(lib.spion_layernorm_backward(ptr(xc), ptr(dy), int(dy.dtype == torch.bfloat16), ptr(w), ptr(mean),
                                               ptr(rstd), ptr(dx), ptr(dw), ptr(db), ptr(ws), M, N,
                                               _lib.current_stream_ptr()), "spion_layernorm_backward")
        return dx, dw, db, None, None


class _AddLayerNormFn(torch.autograd.Function):
    """(x + res, LayerNorm(x + res)) in one pass; the backward adds the gradient that arrives at the sum from its
    other consumers (the next residual connection) to the one through the normalisation in the same kernel."""

    @staticmethod
    def forward(ctx, x, res, weight, bias, eps, out_bf16):
        if not x.is_cuda or x.dtype != torch.float32 or res.dtype not in (torch.float32, torch.bfloat16):
            raise _lib.SpionError("add_norm needs an fp32 CUDA stream and an fp32 or bf16 branch output")
        N = x.shape[-1]
        xc, rc = x.contiguous(), res.contiguous()
        M = xc.numel() // N
        s = torch.empty_like(xc)
        y = torch.empty(xc.shape, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=x.device)
        mean = torch.empty(M, dtype=torch.float32, device=x.device)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        w, b = weight.float().contiguous(), bias.float().contiguous()
        with torch.cuda.device(x.device):
            check(lib.spion_add_layernorm_forward(ptr(xc), ptr(rc), int(rc.dtype == torch.bfloat16), ptr(s), ptr(w), ptr(b),
                                                  ptr(y), int(out_bf16), ptr(mean), ptr(rstd), M, N, float(eps),
                                                  _lib.current_stream_ptr()), "spion_add_layernorm_forward")
        ctx.save_for_backward(s, w, mean, rstd)
        ctx.res_bf16 = rc.dtype == torch.bfloat16
        ctx.set_materialize_grads(False)                          # an unused output arrives as None, not as zeros
        return s, y

    @staticmethod
    def backward(ctx, ds, dy):
        s, w, mean, rstd = ctx.saved_tensors
        N = s.shape[-1]
        M = s.numel() // N
        if dy is None:                                             # the normalised output was not used
            dy = torch.zeros_like(s)
        if dy.dtype not in (torch.float32, torch.bfloat16):
            dy = dy.float()
        dy = dy.contiguous()
        if ds is not None:
            ds = ds.float().contiguous()
        dx = torch.empty_like(s)
        dres = torch.empty(s.shape, dtype=torch.bfloat16, device=s.device) if ctx.res_bf16 else None
        dw = torch.empty(N, dtype=torch.float32, device=s.device)
        db = torch.empty(N, dtype=torch.float32, device=s.device)
        ws = torch.empty(int(lib.spion_layernorm_workspace_floats(N)), dtype=torch.float32, device=s.device)
        with torch.cuda.device(s.device):
            check(lib.spion_add_layernorm_backward(ptr(s), ptr(dy), int(dy.dtype == torch.bfloat16), ptr(w), ptr(mean),
                                                   ptr(rstd), ptr(ds), ptr(dx), ptr(dres), ptr(dw), ptr(db), ptr(ws), M, N,
                                                   _lib.current_stream_ptr()), "spion_add_layernorm_backward")
        return dx, (dres if ctx.res_bf16 else dx), dw, db, None, None


class FusedLayerNorm(nn.Module):
    """Drop-in for ``nn.LayerNorm(dim)`` on fp32 CUDA inputs with dim in SUPPORTED_WIDTHS.

    ``bf16_out=True``: under ``torch.autocast`` the output is bf16 (the dtype the next linear layer casts its
    input to anyway); outside autocast, or with ``bf16_out=False``, it is fp32."""

    def __init__(self, dim: int, eps: float = 1e-5, bf16_out: bool = False):
        super().__init__()
        if dim not in SUPPORTED_WIDTHS:
            raise ValueError(f"FusedLayerNorm: width {dim} not in {SUPPORTED_WIDTHS}")
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps
        self.bf16_out = bf16_out

    def forward(self, x):
        out_bf16 = self.bf16_out and torch.is_autocast_enabled()
        return _LayerNormFn.apply(x.float(), self.weight, self.bias, self.eps, out_bf16)

    def add_norm(self, x, res):
        """``s = x + res`` (x: the fp32 residual stream, res: a branch output, fp32 or bf16) and ``self(s)`` in one
        pass; returns ``(s, self(s))``."""
        out_bf16 = self.bf16_out and torch.is_autocast_enabled()
        if res.dtype not in (torch.float32, torch.bfloat16):
            res = res.float()
        return _AddLayerNormFn.apply(x.float(), res, self.weight, self.bias, self.eps, out_bf16)


# Low-precision copies of linear-layer parameters, refreshed by their owner once per optimizer step with one
# multi-tensor copy (a training loop that casts every weight and bias on every forward spends two small launches per
# layer on it).  id(parameter) -> (weak reference to the parameter, copy).
_SHADOWS: dict = {}


def register_shadows(params, dtype=torch.bfloat16):
    """Create ``dtype`` copies of ``params`` that BiasGradLinear uses instead of casting; returns the list of copies.
    The caller keeps them current with ``refresh_shadows(params, copies)`` after every change of the parameters."""
    import weakref
    for k in [k for k, (r, _) in _SHADOWS.items() if r() is None]:
        del _SHADOWS[k]
    copies = [p.detach().to(dtype) for p in params]
    for p, c in zip(params, copies):
        _SHADOWS[id(p)] = (weakref.ref(p), c)
    return copies


def refresh_shadows(params, copies):
    with torch.no_grad():
        torch._foreach_copy_(copies, [p.detach() for p in params])


def _shadow_or_cast(p, dtype):
    e = _SHADOWS.get(id(p))
    if e is not None and e[0]() is p and e[1].dtype == dtype:
        return e[1]
    return p.to(dtype)


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with the framework's GEMMs; the bias gradient (a column sum over all rows, which the
    framework computes with a slow reduction for bf16 inputs) through spion_column_sums."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        cd = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else x.dtype
        xb, wb, bb = x.to(cd), _shadow_or_cast(weight, cd), _shadow_or_cast(bias, cd)
        with torch.autocast(device_type="cuda", enabled=False):
            y = torch.nn.functional.linear(xb, wb, bb)
        ctx.save_for_backward(xb, wb)
        ctx.in_dtypes = (x.dtype, weight.dtype, bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xb, wb = ctx.saved_tensors
        xd, wd, bd = ctx.in_dtypes
        N, K = wb.shape
        dy2 = dy.reshape(-1, N).contiguous()
        x2 = xb.reshape(-1, K)
        dx = (dy2 @ wb).reshape(xb.shape).to(xd)
        dw = (dy2.t() @ x2).to(wd)
        M = dy2.shape[0]
        if N in SUPPORTED_WIDTHS and dy2.dtype in (torch.float32, torch.bfloat16):
            db = torch.empty(N, dtype=torch.float32, device=dy2.device)
            ws = torch.empty(int(lib.spion_layernorm_workspace_floats(N)), dtype=torch.float32, device=dy2.device)
            with torch.cuda.device(dy2.device):
                check(lib.spion_column_sums(ptr(dy2), int(dy2.dtype == torch.bfloat16), ptr(db), ptr(ws), M, N,
                                            _lib.current_stream_ptr()), "spion_column_sums")
            db = db.to(bd)
        else:
            db = dy2.sum(0).to(bd)
        return dx, dw, db


class BiasGradLinear(nn.Linear):
    """``nn.Linear`` (same parameters, same forward arithmetic) whose backward sums the bias gradient with the
    library's column-sum kernel when the output width is one it serves."""

    def forward(self, x):
        if self.bias is None or not x.is_cuda:
            return super().forward(x)
        return _LinearFn.apply(x, self.weight, self.bias)


class _EmbeddingFn(torch.autograd.Function):
    """Rows of a small table by token id; the weight gradient (a scatter-sum the framework forms by sorting the
    ids) through spion_embedding_backward: table in shared memory, fixed summation order."""

    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.table = (weight.shape, weight.dtype)
        return torch.nn.functional.embedding(ids, weight)

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        (V, N), wd = ctx.table
        return None, _embedding_weight_grad(ids, g, V, N, wd)


def _embedding_weight_grad(ids, g, V, N, wd):
    g2 = g.reshape(-1, N).contiguous()
    idc = ids.reshape(-1).contiguous()
    if idc.data_ptr() % 16:                               # views at odd offsets: the kernel copies 16-byte pieces
        idc = idc.clone()
    if g2.data_ptr() % 16:
        g2 = g2.clone()
    T = idc.numel()
    ws = torch.empty(int(lib.spion_embedding_workspace_floats(T, V, N)), dtype=torch.float32, device=g2.device)
    dW = torch.empty(V, N, dtype=torch.float32, device=g2.device)
    with torch.cuda.device(g2.device):
        check(lib.spion_embedding_backward(ptr(idc), ptr(g2), int(g2.dtype == torch.bfloat16), T, V, N, ptr(dW), ptr(ws),
                                           _lib.current_stream_ptr()), "spion_embedding_backward")
    return dW.to(wd)


class _EmbedPosFn(torch.autograd.Function):
    """tok[ids] + pos[0 .. L-1] for ids [B, L] in one kernel (spion_embedding_forward); backward: the token table's
    gradient through spion_embedding_backward, the position rows' gradient as the sum over the batch."""

    @staticmethod
    def forward(ctx, ids, tok, pos):
        B, L = ids.shape
        V, N = tok.shape
        idc = ids.contiguous()
        out = torch.empty(B, L, N, dtype=torch.float32, device=ids.device)
        with torch.cuda.device(ids.device):
            check(lib.spion_embedding_forward(ptr(idc), ptr(tok), ptr(pos), ptr(out), B * L, L, V, N,
                                              _lib.current_stream_ptr()), "spion_embedding_forward")
        ctx.save_for_backward(idc)
        ctx.shapes = (tok.shape, tok.dtype, pos.shape, pos.dtype)
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        (V, N), td, pshape, pd = ctx.shapes
        B, L = ids.shape
        g = g.float()
        dtok = _embedding_weight_grad(ids, g, V, N, td)
        dpos = torch.zeros(pshape, dtype=torch.float32, device=g.device) if pshape[0] != L else None
        rows = g.reshape(B, L, N).sum(0)
        if dpos is None:
            dpos = rows
        else:
            dpos[:L] = rows
        return None, dtok, dpos.to(pd)


class TokenEmbedding(nn.Embedding):
    """``nn.Embedding`` (same parameter, same forward) whose weight gradient comes from the library's kernel when
    the table is small enough for it (vocab_size * embedding_dim <= 24576, width 32 / 64 / 128 / 256)."""

    def served(self, ids) -> bool:
        V, N = self.weight.shape
        return (ids.is_cuda and ids.dtype == torch.int64 and self.padding_idx is None and self.max_norm is None
                and not self.sparse and not self.scale_grad_by_freq and N in (32, 64, 128, 256) and V * N <= 24576
                and self.weight.dtype == torch.float32)

    def forward(self, ids):
        if not self.served(ids):
            return super().forward(ids)
        return _EmbeddingFn.apply(ids, self.weight)

    def with_positions(self, ids, pos_weight):
        """``self(ids) + pos_weight[:L][None]`` for ids [B, L]: one kernel when the table is served and both tables are
        fp32 rows of the same width (a multiple of 4) on 16-byte boundaries, else the framework's operators."""
        L = ids.shape[-1]
        ok = (ids.dim() == 2 and self.served(ids) and pos_weight.dtype == torch.float32 and pos_weight.is_cuda
              and pos_weight.shape[1] == self.weight.shape[1] and pos_weight.shape[0] >= L
              and pos_weight.is_contiguous() and self.weight.is_contiguous()
              and self.weight.data_ptr() % 16 == 0 and pos_weight.data_ptr() % 16 == 0)
        if not ok:
            return self(ids) + pos_weight[:L][None]
        return _EmbedPosFn.apply(ids, self.weight, pos_weight)
