"""Nefelorn: a decoder-only language model of sequential blocks with Dynamic-Tanh norms before and after every sublayer,
bounded-reach grouped-query attention on key/value rings, and dense or mixture-of-experts feed-forwards.

Structure (every size and constant comes from the configuration):

* token embedding times ``embedding.scale``;
* blocks ``x ← x + n1b(mixer(n1(x)))``, then ``x ← x + n2b(ff(n2(x)))`` (a block may have no feed-forward); every ``n`` is a
  :class:`libai_b200.layers.DynamicTanh`.  Mixers (:class:`libai_b200.layers.RingAttention`):
  ``attention`` — RMS norm over the whole query / key projection, rotary positions whose frequencies may be blended per
  dimension (``rot.scaling``), a chunk mask, a per-head sigmoid output gate, optionally no key/value projections of its own
  (``kv_from``: it reads the cache of another block); ``attention_2`` — rotary positions, then every query / key head divided by
  its root mean square, a sliding window that also keeps the first tokens of the sequence.
  Feed-forwards: ``dense`` — ``W_down gelu(W_up h)``; ``moe`` — :class:`libai_b200.layers.MoEFeedForward`;
* a final Dynamic Tanh, the output projection and ``logits ← cap · tanh(logits / cap)``.

The residual stream, the norms, softmax and the router are fp32 whatever the compute dtype.  Execution is the framework's
generation path for stateful models: packed rows (:class:`~libai_b200.inference.ragged.RaggedBatch`) against a
:class:`~libai_b200.inference.state_cache.SequenceStateCache`; one kernel applies a sublayer's closing norm, the residual sum
and the next sublayer's opening norm.
"""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from libai_b200.config import configurable
from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import DynamicTanh, MoEFeedForward, RingAttention
from libai_b200.layers._param import create_parameter, normal_init, xavier_normal_
from libai_b200.ops import kv_functional as KF
from libai_b200.ops import seq_functional as SF

from .stateful_lm import StatefulCausalLM, _plain


def build_ring_mixer(kind: str, width: int, m: dict, eps: float, layer_idx: int) -> RingAttention:
    """Mixer of one block from its ``type`` and ``mixer`` record."""
    rot = m.get("rot") or {}
    common = dict(scale=m.get("scale"), rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0),
                  rot_scaling=rot.get("scaling"), eps=eps, layer_idx=layer_idx)
    mask = m["mask"]
    if kind == "attention":
        return RingAttention(width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], chunk=mask["size"], qk_norm="full",
                             out_gate=True, kv_source=m.get("kv_from"), **common)
    if kind == "attention_2":
        return RingAttention(width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], window=mask["size"],
                             keep_first=mask.get("keep_first", 0), qk_norm="head_unit", out_gate=False, **common)
    raise ValueError(f"unknown mixer type {kind!r}")


class GeluFF(nn.Module):
    """``W_down act(W_up h)`` without biases."""

    def __init__(self, width, ff, act="gelu", *, layer_idx=0):
        super().__init__()
        self.act = act
        self.up = create_parameter((ff, width), xavier_normal_, layer_idx=layer_idx)
        self.down = create_parameter((width, ff), xavier_normal_, layer_idx=layer_idx)

    def forward(self, h):
        u = KF.linear(h, self.up)
        KF.act_rows(u, u, KF.ACTS[self.act])
        return KF.linear_f32(u, self.down)


class SandwichBlock(nn.Module):
    """``x ← x + n1b(mixer(n1(x)))``, ``x ← x + n2b(ff(n2(x)))`` on the fp32 stream ``x``; the opening norm of a sublayer is
    applied by the kernel that closes the sublayer before it, so a block receives ``h = n1(x)`` and returns the next block's."""

    def __init__(self, width, kind, mixer_cfg, mlp_cfg, eps, *, layer_idx=0):
        super().__init__()
        self.kind, self.width = kind, width
        mk = lambda: DynamicTanh(width, layer_idx=layer_idx)
        self.norm1, self.norm1b = mk(), mk()
        self.mix = build_ring_mixer(kind, width, mixer_cfg, eps, layer_idx)
        self.mlp = None
        if mlp_cfg:
            self.norm2, self.norm2b = mk(), mk()
            kind_ff = mlp_cfg.get("kind", "dense")
            if kind_ff == "dense":
                self.mlp = GeluFF(width, mlp_cfg["ff"], layer_idx=layer_idx)
            elif kind_ff == "moe":
                r = mlp_cfg["router"]
                self.mlp = MoEFeedForward(width, mlp_cfg["expert"]["ff"], r["experts"], r["top"], router_scale=r.get("scale", 1.0),
                                          layer_idx=layer_idx)
            else:
                raise ValueError(f"unknown feed-forward kind {kind_ff!r}")
        self._fused = None

    def _fuse(self):
        w = self.mix.q
        if self._fused is None or self._fused[0].dtype != w.dtype or self._fused[0].device != w.device:
            self._fused = SF.fuse_rows([(n, t.detach()) for n, t in self.mix.input_weights()])
        return self._fused

    def forward(self, x, h, rb, bufs, shared, next_norm):
        """``x`` fp32 stream (updated in place), ``h = norm1(x)``; returns ``next_norm(x)`` (``None`` without one)."""
        w_in, cols = self._fuse()
        dt, dev, T = w_in.dtype, x.device, x.shape[0]
        proj = KF.linear(h, w_in)
        parts = {n: proj[:, lo:lo + size] for n, (lo, size) in cols.items()}
        y = torch.empty(T, self.mix.mix_features, dtype=dt, device=dev)
        self.mix.mix(parts, rb, bufs, y, shared)
        o = KF.linear_f32(y, self.mix.o)
        after = self.norm2 if self.mlp is not None else next_norm
        h = torch.empty(T, self.width, dtype=dt, device=dev) if after is not None else None
        KF.dyt_residual(x, o, post=self.norm1b.triple(), nxt=after.triple() if after is not None else None, h=h)
        if self.mlp is None:
            return h
        pos = cw = None
        if isinstance(self.mlp, MoEFeedForward):
            d, pos, cw = self.mlp(h, graph_safe=rb.single)
        else:
            d = self.mlp(h)
        h = torch.empty(T, self.width, dtype=dt, device=dev) if next_norm is not None else None
        KF.dyt_residual(x, d, post=self.norm2b.triple(), nxt=next_norm.triple() if next_norm is not None else None, h=h, pos=pos, cw=cw)
        return h


class NefelornModel(nn.Module):
    def __init__(self, vocab, width, layers, embedding_scale=1.0, eps=1e-6, initializer_range=0.02):
        super().__init__()
        self.vocab, self.width, self.eps, self.embedding_scale = vocab, width, eps, float(embedding_scale)
        self.embed = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=0)
        self.layers = nn.ModuleList(
            [SandwichBlock(width, lc["type"], lc["mixer"], lc.get("mlp"), eps, layer_idx=i) for i, lc in enumerate(layers)])
        self.final_norm = DynamicTanh(width, layer_idx=-1)
        # a cache is sized for every block that reads it: the longest reach and the most kept-first rows
        for i, blk in enumerate(self.layers):
            src = blk.mix.kv_source
            if src is not None:
                owner = self.layers[src].mix
                if not (0 <= src < i) or owner.kv_source is not None:
                    raise ValueError(f"block {i} reads the keys of block {src}, which must be an earlier block with projections of its own")
                if (owner.kv_heads, owner.dim, owner.vdim) != (blk.mix.kv_heads, blk.mix.dim, blk.mix.vdim):
                    raise ValueError(f"block {i} and block {src} differ in their key / value head sizes")
                owner.cache_masks = owner.cache_masks + [blk.mix.mask]
                owner.ring_len = max(owner.ring_len, blk.mix.reach)
                owner.first_len = max(owner.first_len, blk.mix.keep_first)

    def register_state(self, cache: SequenceStateCache) -> List[int]:
        """One cache entry per block with key/value projections; a block that reads another's keys gets that block's handle."""
        handles: List[int] = []
        for blk in self.layers:
            if blk.mix.kv_source is None:
                kind, shape = blk.mix.state_spec()
                handles.append(cache.register(kind, **shape))
            else:
                handles.append(handles[blk.mix.kv_source])
        return handles

    def forward(self, tokens, rb: RaggedBatch, cache: SequenceStateCache, handles, tap=None):
        """``tokens`` ``[rows]`` int64 packed → the fp32 stream after the last block ``[rows, width]`` (before the final
        norm).  ``tap(run, x)`` is called after every block (diagnostics)."""
        dt = self.embed.dtype
        T = tokens.shape[0]
        x = torch.empty(T, self.width, dtype=torch.float32, device=tokens.device)
        KF.embed_scale(self.embed, tokens, self.embedding_scale, x)
        h = torch.empty(T, self.width, dtype=dt, device=tokens.device)
        if len(self.layers):
            self.layers[0].norm1.rows(x, h)
        shared: dict = {}
        for i, blk in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else None
            h = blk(x, h, rb, cache.buffers(handles[i]), shared, nxt)
            if tap is not None:
                tap(i, x)
        return x


class NefelornForCausalLM(StatefulCausalLM):
    @configurable
    def __init__(self, vocab, width, layers, embedding_scale=1.0, logit_softcap=None, norm_eps=1e-6, initializer_range=0.02, cfg=None):
        super().__init__()
        self.cfg = cfg
        self.logit_softcap = float(logit_softcap) if logit_softcap else None
        self.model = NefelornModel(vocab, width, layers, embedding_scale=embedding_scale, eps=norm_eps,
                                   initializer_range=initializer_range)
        self.head = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=-1)

    @classmethod
    def from_config(cls, cfg):
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        norm, emb = get("norm") or {}, get("embedding") or {}
        return dict(vocab=get("vocab"), width=get("width"), layers=_plain(get("layers")),
                    embedding_scale=emb.get("scale", 1.0) if hasattr(emb, "get") else 1.0, logit_softcap=get("logit_softcap"),
                    norm_eps=norm.get("eps", 1e-6) if hasattr(norm, "get") else 1e-6,
                    initializer_range=get("initializer_range") or 0.02, cfg=cfg)

    @torch.no_grad()
    def step_device(self, tokens, rb: RaggedBatch, logits_rows=None, tap=None):
        """The device work of :meth:`step` alone (kernel launches only, no host-side bookkeeping): this is what a CUDA graph of a
        single-token step captures."""
        cache = self.state_cache()
        x = self.model(tokens, rb, cache, self._handles, tap=tap)
        if logits_rows is not None:
            x = x.index_select(0, logits_rows)
        h = torch.empty(x.shape, dtype=self.head.dtype, device=x.device)
        self.model.final_norm.rows(x, h)
        logits = KF.linear_f32(h, self.head)
        if self.logit_softcap:
            KF.softcap(logits, self.logit_softcap)
        return logits
