"""Synthetic-data training harness around the attention path (stock torch.nn everywhere else).

The encoder, task heads and training loop of the reference (models/model_transformer.py,
models/model_LRA.py, main_conv_ff.py:132-318) are not part of the accelerated path; this file
is the thin stand-in that lets the end-to-end benchmark configs run: a 2-layer pre-LN encoder
classifier (single or dual tower) whose attention is ``spion_b200.attention.Attention``, with
the reference's phase structure -- dense warm-up steps that return the per-layer mean
attention map, pattern discovery, then sparse steps -- and data parallelism from
``spion_b200.dp``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import dp
from .attention import Attention
from .pattern import discover_layers


def task_config(task: str, batch_size: int, native: bool = True, dtype: str = "fp32"):
    """Model dictionaries with the reference's keys and values (config.py) for the three
    benchmark shapes; max_seq_len is rounded up to a power of two as main_conv_ff.py:385 does."""
    base = dict(learn_pos_emb=True, tied_weights=False, embedding_dim=64, transformer_dim=64,
                transformer_hidden_dim=128, head_dim=32, num_head=2, num_layers=2, dropout_prob=0.1,
                attention_dropout=0.1, pooling_mode="MEAN", mixed_precision=(dtype == "bf16"),
                batch_size=batch_size, native=native, dtype=dtype)
    if task == "image":
        base.update(task="lra-image", vocab_size=256, max_seq_len=1024, num_classes=10, block_size=32,
                    threshold=0.96, density=0.04, dual=False)
    elif task == "text":
        base.update(task="lra-text", vocab_size=256, max_seq_len=4096, num_classes=2, block_size=64,
                    threshold=0.99, density=0.03, dual=False)
    elif task == "retrieval":
        base.update(task="lra-retrieval", vocab_size=256, max_seq_len=4096, num_classes=2, block_size=64,
                    threshold=0.99, density=0.021, dual=True)
    else:
        raise ValueError(task)
    return base


def make_norm(config, feeds_linear: bool):
    """LayerNorm of the encoder: the library's kernels when the configuration asks for the native path and the
    width is one they serve, else torch.nn.LayerNorm (what the reference uses).  feeds_linear: the output only
    goes into linear layers, so under mixed precision it may be bf16 straight away."""
    from .layernorm import SUPPORTED_WIDTHS, FusedLayerNorm
    dim = config["transformer_dim"]
    if config.get("native") and config.get("fused_layernorm", True) and dim in SUPPORTED_WIDTHS:
        return FusedLayerNorm(dim, bf16_out=feeds_linear)
    return nn.LayerNorm(dim)


class Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        Embedding = nn.Embedding
        if config.get("native") and config.get("fused_embedding_grad", True):
            from .layernorm import TokenEmbedding as Embedding      # same parameter and forward; own weight gradient
        self.tok = Embedding(config["vocab_size"], config["embedding_dim"])
        self.pos = nn.Embedding(config["max_seq_len"], config["embedding_dim"])
        nn.init.normal_(self.tok.weight, std=0.02)
        nn.init.normal_(self.pos.weight, std=0.02)
        self.drop = nn.Dropout(config["dropout_prob"])

    def forward(self, ids):
        # positions 0 .. L-1 are a slice of the table: the same values as the lookup self.pos(arange(L)) of the
        # reference (models/model_transformer.py), with a plain sum over the batch as backward instead of the
        # sort-based embedding backward
        if hasattr(self.tok, "with_positions"):
            return self.drop(self.tok.with_positions(ids, self.pos.weight))         # gather and sum in one kernel
        return self.drop(self.tok(ids) + self.pos.weight[:ids.shape[1]][None])


class TransformerLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        dim, hid, p = config["transformer_dim"], config["transformer_hidden_dim"], config["dropout_prob"]
        self.norm1 = make_norm(config, True)
        self.mha = Attention(config)
        self.dropout1 = nn.Dropout(p)
        self.norm2 = make_norm(config, True)
        Linear = nn.Linear
        if config.get("native") and config.get("fused_bias_grad", True):
            from .layernorm import BiasGradLinear as Linear
        self.mlpblock = nn.Sequential(Linear(dim, hid), nn.GELU(), nn.Dropout(p), Linear(hid, dim), nn.Dropout(p))

    def forward(self, X, mask, mat=None):
        out, attn = self.mha(self.norm1(X), mask, mat)
        X = self.dropout1(out) + X
        return self.mlpblock(self.norm2(X)) + X, attn

    def forward_add_norm(self, X, Xn, mask, mat, next_norm):
        """The same layer with each residual addition done inside the normalisation that follows it
        (FusedLayerNorm.add_norm): ``Xn`` is ``self.norm1(X)``, already formed by the previous stage; returns the
        layer's output together with ``next_norm`` of it (the next layer's norm1, or the encoder's final norm)."""
        out, attn = self.mha(Xn, mask, mat)
        X, n2 = self.norm2.add_norm(X, self.dropout1(out))
        X, nn_ = next_norm.add_norm(X, self.mlpblock(n2))
        return X, nn_, attn


class Encoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embeddings = Embeddings(config)
        self.layers = nn.ModuleList(TransformerLayer(config) for _ in range(config["num_layers"]))
        self.norm = make_norm(config, False)
        from .layernorm import FusedLayerNorm
        self.add_norm = bool(config.get("fused_add_norm", True)) and isinstance(self.norm, FusedLayerNorm)

    def forward(self, ids, mask, mat_lst=None, is_attn=False):
        from .pattern import mean_attention_map
        X = self.embeddings(ids)
        maps = []
        if self.add_norm and mat_lst is not None:
            # sparse phase: residual additions inside the normalisation kernels
            Xn = self.layers[0].norm1(X)
            for i, layer in enumerate(self.layers):
                nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else self.norm
                X, Xn, _ = layer.forward_add_norm(X, Xn, mask, mat_lst[0][i], nxt)
            return Xn * mask[:, :, None], maps
        for i, layer in enumerate(self.layers):
            if mat_lst is None:
                X, attn = layer(X, mask)
                if is_attn and layer.mha.native:
                    maps.append(layer.mha.attn.mean_attention_map(attn))      # from block tiles
                elif is_attn:
                    # attn is the permuted view of the S^T-stored tensor: its base is contiguous
                    maps.append(mean_attention_map(attn.permute(0, 1, 3, 2), transposed_storage=True))
            else:
                X, _ = layer(X, mask, mat_lst[0][i])
        return self.norm(X) * mask[:, :, None], maps


class Classifier(nn.Module):
    """Single tower (image / text) or dual tower sharing one encoder (retrieval)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.dual = bool(config.get("dual", False))
        self.batch_towers = bool(config.get("batch_towers", True)) and bool(config.get("native"))
        self.amp = bool(config.get("mixed_precision", False))
        self.model = Encoder(config)
        dim, hid = config["transformer_dim"], config["transformer_hidden_dim"]
        self.head = nn.Sequential(nn.Linear(dim * (4 if self.dual else 1), hid), nn.ReLU(),
                                  nn.Linear(hid, config["num_classes"]))

    def forward(self, ids, label, mat_lst=None, is_attn=False):
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16, enabled=self.amp):
            if self.dual and mat_lst is not None and self.batch_towers:
                # sparse phase: both sequences of a pair go through the shared encoder as one batch of 2 B
                # (the reference calls the encoder twice, models/model_LRA.py; same weights, same arithmetic
                # per sequence, half the kernel launches and no second accumulation of the weight gradients)
                both = torch.cat([ids[0], ids[1]], 0)
                t, maps = self.model(both, (both != 0).float(), mat_lst, False)
                nb = ids[0].shape[0]
                x0, x1 = t[:nb].mean(1), t[nb:].mean(1)
                scores = self.head(torch.cat([x0, x1, x0 * x1, x0 - x1], dim=-1))
            elif self.dual:
                m0, m1 = (ids[0] != 0).float(), (ids[1] != 0).float()        # models/dataset_LRA.py:34
                t0, maps = self.model(ids[0], m0, mat_lst, is_attn)
                t1, _ = self.model(ids[1], m1, mat_lst, False)
                x0, x1 = t0.mean(1), t1.mean(1)
                scores = self.head(torch.cat([x0, x1, x0 * x1, x0 - x1], dim=-1))
            else:
                mask = (ids != 0).float()
                t, maps = self.model(ids, mask, mat_lst, is_attn)
                scores = self.head(t.mean(1))
            loss = nn.functional.cross_entropy(scores.float(), label)
        return loss, maps


class Trainer:
    """dense step(s) -> discover -> sparse steps, with one flat-bucket all-reduce per step."""

    def __init__(self, config, lr: float = 1e-4, device=None, seed: int = 0):
        self.config = config
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        torch.manual_seed(seed)                      # identical initial weights on every rank
        self.model = Classifier(config).to(self.device)
        self.bucket = dp.FlatGradBucket(self.model.parameters())
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=0.0, capturable=True, fused=True)
        self.mat_lst = None
        self.patterns = None
        self._graph = None
        # bf16 copies of the linear layers' parameters, refreshed once per optimizer step (mixed precision only)
        self._shadow = None
        if config.get("native") and config.get("mixed_precision") and config.get("shadow_weights", True):
            from .layernorm import BiasGradLinear, register_shadows
            ps = [p for m in self.model.modules() if isinstance(m, BiasGradLinear) for p in (m.weight, m.bias)]
            if ps:
                self._shadow = (ps, register_shadows(ps))
        self.allreduce_events = None     # set to a list to collect (start, end) CUDA events around the gradient all-reduce

    def step(self, ids, label, is_attn=False):
        self.bucket.zero()
        loss, maps = self.model(ids, label, self.mat_lst, is_attn)
        loss.backward()
        if self.allreduce_events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.bucket.allreduce_mean()
            e1.record()
            self.allreduce_events.append((e0, e1))
        else:
            self.bucket.allreduce_mean()
        torch.nn.utils.clip_grad_value_(self.model.parameters(), 1.0)   # main_conv_ff.py:186
        self.opt.step()
        self._refresh_shadows()
        return loss.detach(), maps

    def _refresh_shadows(self):
        if self._shadow is not None:
            from .layernorm import refresh_shadows
            refresh_shadows(*self._shadow)

    def capture_sparse_step(self, ids, label, warmup: int = 3):
        """Record one sparse step as CUDA graphs: the step is a few hundred small launches, so replaying it
        removes most of the host time (at 8 samples per GPU the eager step is host-bound).  The library's calls
        are plain stream-ordered launches with caller-owned buffers, which is what capture needs.
        One rank: a single graph (forward, backward, clipping, optimizer).  Several ranks: two graphs --
        forward + backward, and clipping + optimizer -- with the gradient all-reduce issued eagerly between
        the two replays, so that no collective is ever part of a capture."""
        if self.mat_lst is None:
            raise RuntimeError("capture the step after discover()")
        multi = dp.world_size() > 1
        dual = isinstance(ids, (tuple, list))
        self._g_ids = tuple(t.clone() for t in ids) if dual else ids.clone()
        self._g_lab = label.clone()
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step(self._g_ids, self._g_lab)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        self._graph_opt = None
        if not multi:
            with torch.cuda.graph(self._graph):
                self._g_loss, _ = self.step(self._g_ids, self._g_lab)
            return self._graph
        # other threads of the process (the collective library's watchdog) may query events while this thread
        # captures: only this thread's calls belong to the capture
        with torch.cuda.graph(self._graph, capture_error_mode="thread_local"):
            self.bucket.zero()
            loss, _ = self.model(self._g_ids, self._g_lab, self.mat_lst, False)
            loss.backward()
            self._g_loss = loss.detach()
        self._graph_opt = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph_opt, capture_error_mode="thread_local"):
            torch.nn.utils.clip_grad_value_(self.model.parameters(), 1.0)
            self.opt.step()
            self._refresh_shadows()
        return self._graph

    def step_graph(self, ids, label):
        """Replay the captured step on new inputs (copied into the graph's static buffers)."""
        if isinstance(ids, (tuple, list)):
            for dst, src in zip(self._g_ids, ids):
                dst.copy_(src, non_blocking=True)
        else:
            self._g_ids.copy_(ids, non_blocking=True)
        self._g_lab.copy_(label, non_blocking=True)
        ev = None
        if self.allreduce_events is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
        self._graph.replay()
        if ev:
            ev[1].record()
        if self._graph_opt is not None:
            self.bucket.allreduce_mean()                      # eager, between the two replays
            if ev:
                ev[2].record()
            self._graph_opt.replay()
        if ev:
            if self._graph_opt is None:
                ev[2].record()
            ev[3].record()
            self.allreduce_events.append(tuple(ev))
        return self._g_loss

    def discover(self, maps, threshold=None):
        cfg = dict(self.config)
        if threshold is not None:
            cfg["threshold"] = threshold
        bs = cfg["block_size"]

        def disc(A):
            from .pattern import discover_pattern
            return discover_pattern(A, bs, cfg["threshold"]).mat

        masks = dp.agree_on_masks(maps, disc)
        mats = torch.stack([m.to(torch.float32) for m in masks], 0)
        self.mat_lst = torch.stack([mats, mats, mats, mats], 0)          # main_conv_ff.py:298-299
        if self.model.dual and self.model.batch_towers:
            cfg["batch_size"] = 2 * cfg["batch_size"]                   # the sparse layers see both towers at once
        for layer in self.model.model.layers:
            layer.mha.reconstruct_for_blocksparse(cfg)
        return self.mat_lst
