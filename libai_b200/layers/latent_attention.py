"""Sliding-window attention whose keys and values are up-projections of one cached low-rank latent per token.

``c_q = rmsnorm(W_dq h)``, ``q = W_uq c_q``; ``c = rmsnorm(W_dkv h)`` is the only thing cached; per head ``k = W_uk c``,
``v = W_uv c``; ``score = (q·k)·scale``; position ``i`` sees ``j`` with ``0 ≤ i − j < window``; plain softmax; head ``h`` of
the result is multiplied by ``sigmoid(W_g h)_h``; ``W_o`` mixes the heads.  No positional signal enters the scores.

Prompts expand keys and values for the rows a step needs (one GEMM on ``[cached window | new latents]``) and run the
windowed softmax kernel; single-token steps use the absorbed form — ``q`` is pulled through ``W_uk`` so the scores and the
weighted sum run on the cached latents themselves and ``W_uv`` is applied to the result — which reads ``window·C`` numbers
per sequence instead of expanding ``window`` keys and values.  State per sequence: a ring of the last ``window`` latents
(:class:`libai_b200.inference.state_cache.SequenceStateCache`, kind ``latent``).
"""
from __future__ import annotations

import torch
from torch import nn

from libai_b200.ops import seq_functional as SF

from ._param import create_parameter, ones_, xavier_normal_


class LatentAttention(nn.Module):
    def __init__(self, width, heads, dim, vdim, q_rank, kv_rank, window, scale=None, eps=1e-6, out_gate=True,
                 init_method=xavier_normal_, absorbed_decode=True, *, layer_idx=0):
        super().__init__()
        self.width, self.heads, self.dim, self.vdim, self.q_rank, self.kv_rank = width, heads, dim, vdim, q_rank, kv_rank
        self.window, self.scale, self.eps = int(window), float(scale if scale is not None else dim ** -0.5), eps
        self.absorbed_decode = absorbed_decode
        mk = lambda shape, init=init_method: create_parameter(shape, init, layer_idx=layer_idx)
        self.dq, self.dq_norm, self.uq = mk((q_rank, width)), mk((q_rank,), ones_), mk((heads * dim, q_rank))
        self.dkv, self.dkv_norm = mk((kv_rank, width)), mk((kv_rank,), ones_)
        self.uk, self.uv = mk((heads * dim, kv_rank)), mk((heads * vdim, kv_rank))
        self.g = mk((heads, width)) if out_gate else None
        self.o = mk((width, heads * vdim))
        self._ukv = self._uk3 = self._uv3 = None

    @property
    def mix_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self):
        return "latent", dict(ring_len=self.window, channels=self.kv_rank)

    def input_weights(self):
        out = [("dq", self.dq), ("dkv", self.dkv)]
        if self.g is not None:
            out.append(("g", self.g))
        return out

    def output_weight(self):
        return self.o

    def _derived(self):
        if self._ukv is None or self._ukv.dtype != self.uk.dtype or self._ukv.device != self.uk.device:
            self._ukv = torch.cat([self.uk, self.uv], 0).detach().contiguous()
            self._uk3 = self.uk.detach().view(self.heads, self.dim, self.kv_rank)
            self._uv3 = self.uv.detach().view(self.heads, self.vdim, self.kv_rank)

    def mix(self, parts, rb, bufs, y):
        self._derived()
        T, dt, dev = parts["dq"].shape[0], parts["dq"].dtype, parts["dq"].device
        cq = torch.empty(T, self.q_rank, dtype=dt, device=dev)
        SF.rms_norm_rows(parts["dq"], self.dq_norm, offset=0.0, eps=self.eps, out=cq)
        c = torch.empty(T, self.kv_rank, dtype=dt, device=dev)
        SF.rms_norm_rows(parts["dkv"], self.dkv_norm, offset=0.0, eps=self.eps, out=c)
        q = SF.linear(cq, self.uq)
        gate = parts.get("g")
        ring = bufs["ring"]
        H, D, V = self.heads, self.dim, self.vdim
        if rb.single and self.absorbed_decode:
            qa = torch.einsum("bhd,hdc->bhc", q.view(T, H, D).float(), self._uk3.float())
            lat = SF.latent_decode(qa.contiguous(), ring, c, rb, self.window, self.scale)
            SF.head_gate(torch.einsum("bhc,hvc->bhv", lat, self._uv3.float()).contiguous(), gate, y, H, V)
        else:
            kv = SF.linear(SF.latent_gather(ring, c, rb, self.window), self._ukv)
            SF.window_attention(q, kv, gate, rb, y, H, D, V, self.window, self.scale)
        SF.latent_write(ring, c, rb)
        return y

    def forward(self, h, rb, bufs):
        parts = {name: SF.linear(h, w) for name, w in self.input_weights()}
        y = torch.empty(h.shape[0], self.mix_features, dtype=h.dtype, device=h.device)
        return SF.linear(self.mix(parts, rb, bufs, y), self.o)
