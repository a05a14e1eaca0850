"""Bumodra: a decoder-only language model of parallel blocks whose sequence mixers carry per-sequence state.

Structure (every size comes from the configuration):

* token embedding followed by a zero-centred RMS norm; ``x0`` denotes its output;
* a list of blocks, each ``x ← x + mixer(n(x)) + ff(n(x))`` with ONE zero-centred RMS norm ``n`` feeding both branches (a block
  may have no feed-forward).  The mixer is one of ``latent_attention`` (:class:`libai_b200.layers.LatentAttention`:
  sliding-window attention on cached low-rank latents, per-head sigmoid output gate), ``delta``
  (:class:`libai_b200.layers.GatedDeltaMixer`, one decay per head, SiLU gate) or ``channel_delta`` (same rule, one decay
  per head and key channel and a sigmoid gate, both through low-rank pairs).  The feed-forward is ``W_down relu(W_up h)²``;
* an optional loop: blocks ``start … stop−1`` run ``times`` times in a row with the same weights, each pass with its own
  state, and every pass is entered through ``x ← W_in [x; x0]``;
* a final zero-centred RMS norm and the output projection.

The residual stream, the norms, the softmax and everything inside the recurrences are fp32 whatever the compute dtype.

Execution.  The model runs on packed rows (:class:`libai_b200.inference.ragged.RaggedBatch`) against a
:class:`libai_b200.inference.state_cache.SequenceStateCache`; :meth:`BumodraForCausalLM.step` is the one step function —
``forward`` (and through it ``Generator.generate``), the request scheduler and the trace runner all call it.  A block is
two GEMMs around its mixer: every matrix that reads the normed input (mixer projections and ``W_up``) is one product, and
``W_o`` and ``W_down`` are one product on ``[mixer output | relu²]`` that accumulates straight into the fp32 residual.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from libai_b200.config import configurable
from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import GatedDeltaMixer, LatentAttention, RMSLayerNorm
from libai_b200.layers._param import create_parameter, normal_init, xavier_normal_
from libai_b200.ops import seq_functional as SF

from .stateful_lm import StatefulCausalLM, _plain

_FF_ACTS = {"relu2": SF.ACT_RELU2, "silu": SF.ACT_SILU, "gelu_tanh": SF.ACT_GELU_TANH}


def build_mixer(kind: str, width: int, m: dict, eps: float, layer_idx: int):
    """Mixer of one block from its ``type`` and ``mixer`` record."""
    if kind == "latent_attention":
        return LatentAttention(width, m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["mask"]["size"],
                               scale=m.get("scale"), eps=eps, out_gate=True, layer_idx=layer_idx)
    if kind == "delta":
        return GatedDeltaMixer(width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], decay="head", gate="silu",
                               eps=eps, layer_idx=layer_idx)
    if kind == "channel_delta":
        return GatedDeltaMixer(width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], decay="channel",
                               decay_rank=m["decay_rank"], gate="sigmoid_lowrank", gate_rank=m["gate_rank"], eps=eps,
                               layer_idx=layer_idx)
    raise ValueError(f"unknown mixer type {kind!r}")


class DenseFF(nn.Module):
    """``W_down act(W_up h)`` without biases; inside a parallel block only its weights are used (fused products)."""

    def __init__(self, width, ff, act="relu2", *, layer_idx=0):
        super().__init__()
        self.act = act
        self.up = create_parameter((ff, width), xavier_normal_, layer_idx=layer_idx)
        self.down = create_parameter((width, ff), xavier_normal_, layer_idx=layer_idx)

    def forward(self, h):
        u = SF.linear(h, self.up)
        a = torch.empty_like(u)
        SF.slice_act(u, a, _FF_ACTS[self.act])
        return SF.linear(a, self.down)


class ParallelBlock(nn.Module):
    """``x ← x + mixer(n(x)) + ff(n(x))`` on the fp32 stream ``x``."""

    def __init__(self, width, kind, mixer_cfg, mlp_cfg, eps, *, layer_idx=0):
        super().__init__()
        self.kind, self.width = kind, width
        self.norm1 = RMSLayerNorm(width, eps=eps, zero_centered=True, layer_idx=layer_idx)
        self.mix = build_mixer(kind, width, mixer_cfg, eps, layer_idx)
        self.mlp = None
        if mlp_cfg:
            if mlp_cfg.get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind {mlp_cfg.get('kind')!r}")
            self.mlp = DenseFF(width, mlp_cfg["ff"], layer_idx=layer_idx)
        self._fused = None

    def _fuse(self):
        w = self.norm1.weight
        if self._fused is None or self._fused[0].dtype != w.dtype or self._fused[0].device != w.device:
            ins = [(n, t.detach()) for n, t in self.mix.input_weights()]
            outs = [("mix", self.mix.output_weight().detach())]
            if self.mlp is not None:
                ins.append(("up", self.mlp.up.detach()))
                outs.append(("ff", self.mlp.down.detach()))
            self._fused = SF.fuse_rows(ins) + SF.fuse_cols(outs)
        return self._fused

    def forward(self, x, rb, bufs):
        w_in, cols, w_out, kcols = self._fuse()
        dt = w_in.dtype
        h = torch.empty(x.shape, dtype=dt, device=x.device)
        self.norm1.rows(x, h)
        proj = SF.linear(h, w_in)
        parts = {n: proj[:, lo:lo + size] for n, (lo, size) in cols.items()}
        cat = torch.zeros(x.shape[0], w_out.shape[1], dtype=dt, device=x.device) if w_out.shape[1] != sum(
            s for _, s in kcols.values()) else torch.empty(x.shape[0], w_out.shape[1], dtype=dt, device=x.device)
        lo, size = kcols["mix"]
        self.mix.mix(parts, rb, bufs, cat[:, lo:lo + size])
        if self.mlp is not None:
            lo, size = kcols["ff"]
            SF.slice_act(parts["up"], cat[:, lo:lo + size], _FF_ACTS[self.mlp.act])
        return SF.linear_accumulate(x, cat, w_out)


class BumodraModel(nn.Module):
    def __init__(self, vocab, width, layers, loop=None, eps=1e-6, initializer_range=0.02):
        super().__init__()
        self.vocab, self.width, self.eps = vocab, width, eps
        self.loop = dict(loop) if loop else None
        self.embed = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=0)
        self.embed_norm = RMSLayerNorm(width, eps=eps, zero_centered=True, layer_idx=0)
        self.layers = nn.ModuleList(
            [ParallelBlock(width, lc["type"], lc["mixer"], lc.get("mlp"), eps, layer_idx=i) for i, lc in enumerate(layers)])
        self.loop_in = create_parameter((width, 2 * width), xavier_normal_, layer_idx=0) if self.loop else None
        self.final_norm = RMSLayerNorm(width, eps=eps, zero_centered=True, layer_idx=-1)
        # (block index, enters a pass) for every block run, in execution order
        n = len(layers)
        if self.loop:
            a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            assert 0 <= a < b <= n and times >= 1
            self.runs = [(i, False) for i in range(a)]
            for _ in range(times):
                self.runs += [(i, i == a) for i in range(a, b)]
            self.runs += [(i, False) for i in range(b, n)]
        else:
            self.runs = [(i, False) for i in range(n)]

    def register_state(self, cache: SequenceStateCache) -> List[int]:
        handles = []
        for i, _ in self.runs:
            kind, shape = self.layers[i].mix.state_spec()
            handles.append(cache.register(kind, **shape))
        return handles

    def forward(self, tokens, rb: RaggedBatch, cache: SequenceStateCache, handles, tap=None):
        """``tokens`` ``[rows]`` int64 packed → the fp32 stream after the last block ``[rows, width]`` (before the final
        norm).  ``tap(run, x)`` is called after every block run (diagnostics)."""
        dt = self.embed.dtype
        x = torch.empty(tokens.shape[0], self.width, dtype=torch.float32, device=tokens.device)
        self.embed_norm.rows(self.embed, x, ids=tokens)
        x0 = None
        if self.loop:
            x0 = x.to(dt, copy=True)             # the blocks update x in place
        for run, (i, enters) in enumerate(self.runs):
            if enters:
                x = SF.linear(torch.cat([x.to(dt), x0], 1), self.loop_in).float()
            x = self.layers[i](x, rb, cache.buffers(handles[run]))
            if tap is not None:
                tap(run, x)
        return x


class BumodraForCausalLM(StatefulCausalLM):
    @configurable
    def __init__(self, vocab, width, layers, loop=None, norm_eps=1e-6, initializer_range=0.02, cfg=None):
        super().__init__()
        self.cfg = cfg
        self.model = BumodraModel(vocab, width, layers, loop=loop, eps=norm_eps, initializer_range=initializer_range)
        self.head = create_parameter((vocab, width), normal_init(initializer_range), layer_idx=-1)

    @classmethod
    def from_config(cls, cfg):
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        norm = get("norm") or {}
        return dict(vocab=get("vocab"), width=get("width"), layers=_plain(get("layers")), loop=_plain(get("loop")),
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
        return SF.linear(h, self.head).float()
