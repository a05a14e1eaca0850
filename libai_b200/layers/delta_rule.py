"""Gated delta-rule sequence mixer (a linear-attention layer with an fp32 matrix state per head).

Per head, with the state ``S`` ``[dim, vdim]`` and, for every token, a unit-length key ``k``, a unit-length query ``q``
scaled by ``dim^-1/2``, a value ``v``, a write strength ``β = sigmoid(W_b h)`` and a decay ``g``::

    S ← diag(g) S;   u = β (v − Sᵀk);   S ← S + k uᵀ;   o = Sᵀq

``q, k, v`` are projections of the layer input followed by a short causal per-channel convolution and SiLU; query / key
heads may be shared by groups of value heads.  ``decay="head"``: one ``g = exp(−exp(A_log) · softplus(W_a h + dt_bias))``
per head; ``decay="channel"``: one per head and key channel, its logits going through a low-rank pair ``W_a2 W_a1``.  The
read-out is RMS-normalised per head, scaled by a weight shared by the heads and gated by ``silu(W_g h)`` (``gate="silu"``) or
``sigmoid(W_g2 W_g1 h)`` (``gate="sigmoid_lowrank"``), then projected by ``W_o``.  State per sequence: ``S`` and the last
``taps − 1`` inputs of the convolutions (:class:`libai_b200.inference.state_cache.SequenceStateCache`, kind ``recurrent``).
"""
from __future__ import annotations

import torch
from torch import nn

from libai_b200.ops import seq_functional as SF

from ._param import create_parameter, normal_init, ones_, xavier_normal_, zeros_


class GatedDeltaMixer(nn.Module):
    def __init__(self, width, heads, kv_heads, dim, vdim, conv_taps, decay="head", decay_rank=None, gate="silu", gate_rank=None,
                 eps=1e-6, init_method=xavier_normal_, *, layer_idx=0):
        super().__init__()
        assert decay in ("head", "channel") and gate in ("silu", "sigmoid_lowrank") and heads % kv_heads == 0
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = width, heads, kv_heads, dim, vdim, conv_taps
        self.decay, self.gate, self.eps = decay, gate, eps
        mk = lambda shape, init=init_method: create_parameter(shape, init, layer_idx=layer_idx)
        self.q, self.k, self.v = mk((kv_heads * dim, width)), mk((kv_heads * dim, width)), mk((heads * vdim, width))
        conv_init = normal_init(0.3)
        self.q_conv, self.k_conv = mk((kv_heads * dim, conv_taps), conv_init), mk((kv_heads * dim, conv_taps), conv_init)
        self.v_conv = mk((heads * vdim, conv_taps), conv_init)
        self.b = mk((heads, width))
        self.A_log = mk((heads,), zeros_)
        self.norm = mk((vdim,), ones_)
        if decay == "head":
            self.a, self.dt_bias = mk((heads, width)), mk((heads,), zeros_)
        else:
            self.a1, self.a2 = mk((decay_rank, width)), mk((heads * dim, decay_rank))
            self.dt_bias = mk((heads * dim,), zeros_)
        if gate == "silu":
            self.g = mk((heads * vdim, width))
        else:
            self.g1, self.g2 = mk((gate_rank, width)), mk((heads * vdim, gate_rank))
        self.o = mk((width, heads * vdim))
        self._conv_w = None

    # ------------------------------------------------------------------ protocol of the parallel block
    @property
    def mix_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self):
        return "recurrent", dict(heads=self.heads, dim=self.dim, vdim=self.vdim, taps=self.taps,
                                 conv_channels=2 * self.kv_heads * self.dim + self.heads * self.vdim)

    def input_weights(self):
        """Matrices applied to the layer input; ``qkv`` stays one segment so that the convolution sees adjacent columns."""
        out = [("qkv", torch.cat([self.q, self.k, self.v], 0)), ("b", self.b)]
        out.append(("a", self.a) if self.decay == "head" else ("a1", self.a1))
        out.append(("g", self.g) if self.gate == "silu" else ("g1", self.g1))
        return out

    def output_weight(self):
        return self.o

    def mix(self, parts, rb, bufs, y):
        """From the projections of the layer input (``parts``: name → column view) to the gated, normalised read-out written
        into ``y`` ``[tokens, heads·vdim]`` (the input of ``W_o``)."""
        if self._conv_w is None or self._conv_w.dtype != self.q_conv.dtype or self._conv_w.device != self.q_conv.device:
            self._conv_w = torch.cat([self.q_conv, self.k_conv, self.v_conv], 0).detach().contiguous()
        qkv = parts["qkv"]
        conv = torch.empty(qkv.shape[0], qkv.shape[1], dtype=qkv.dtype, device=qkv.device)
        SF.short_conv(qkv, self._conv_w, bufs["tail"], rb, conv)
        kd = self.kv_heads * self.dim
        a = parts["a"] if self.decay == "head" else SF.linear(parts["a1"], self.a2)
        o = SF.delta_scan(conv, kd, 2 * kd, a, parts["b"], self.A_log, self.dt_bias, bufs["S"], rb, self.kv_heads,
                          self.decay == "channel")
        if self.gate == "silu":
            SF.gated_rmsnorm(o, parts["g"], self.norm, self.eps, SF.GATE_SILU, y, self.heads, self.vdim)
        else:
            SF.gated_rmsnorm(o, SF.linear(parts["g1"], self.g2), self.norm, self.eps, SF.GATE_SIGMOID, y, self.heads, self.vdim)
        return y

    def forward(self, h, rb, bufs):
        """Unfused form: ``h`` ``[tokens, width]`` packed rows → ``[tokens, width]``."""
        parts = {name: SF.linear(h, w) for name, w in self.input_weights()}
        y = torch.empty(h.shape[0], self.mix_features, dtype=h.dtype, device=h.device)
        return SF.linear(self.mix(parts, rb, bufs, y), self.o)
