"""Operators on ragged batches with per-sequence state (``csrc/seq_mixers.cu``): zero-centred RMS norms, short causal
convolutions with carried tails, the gated delta rule and sliding-window attention over cached latents.

Every operator takes the step's :class:`~libai_b200.inference.ragged.RaggedBatch` (packed rows, slots, past lengths).  On a
CUDA device the native kernels run (a missing extension is an error, there is no fallback); on the CPU the same operators
are plain PyTorch, sequence by sequence, which is what the CPU tests and the gloo plumbing use.  Arithmetic that feeds a
norm, a softmax or a recurrence is fp32 in both.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import count_launch, impl, load_seq_ext

ACT_COPY, ACT_RELU2, ACT_SILU, ACT_GELU_TANH = 0, 1, 2, 3
GATE_SILU, GATE_SIGMOID = 0, 1


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and impl() == "native"


# ----------------------------------------------------------------------------------------------------------------- norms
def rms_norm_rows(x, w, *, offset: float, eps: float, out, ids=None):
    """``out[r] = x[r] / sqrt(mean(x[r]²) + eps) · (offset + w)`` over 2-D row views (``x`` fp32 or the compute dtype;
    with ``ids`` row r of the output reads row ``ids[r]`` of ``x`` — embedding lookup and norm in one pass)."""
    if _native(x):
        count_launch()
        load_seq_ext().rmsnorm(x, ids, w, float(offset), float(eps), out)
        return out
    xr = (x if ids is None else x[ids]).float()
    y = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps) * (offset + w.float())
    out.copy_(y)
    return out


def slice_act(inp, out, act: int):
    """``out = act(inp)`` between column slices of two row-major matrices (copy / relu² / silu / gelu_tanh)."""
    if _native(inp):
        count_launch()
        load_seq_ext().slice_act(inp, out, act)
        return out
    v = inp.float()
    if act == ACT_RELU2:
        v = torch.relu(v) ** 2
    elif act == ACT_SILU:
        v = F.silu(v)
    elif act == ACT_GELU_TANH:
        v = F.gelu(v, approximate="tanh")
    out.copy_(v)
    return out


def linear_accumulate(x32, a, w):
    """``x32 += a @ wᵀ`` with the fp32 residual stream as the accumulator: on the tcgen05 GEMM the product is added to
    ``x32`` by the epilogue (fp32 ``red.add``), so the residual sum never passes through 16 bits."""
    from . import load_ext, use_native

    if (a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and use_native(a) and a.stride(-1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and w.shape[0] % 8 == 0 and x32.stride(0) % 4 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.shape[0] > 0):
        if _tcgen05_gemm(a, w, x32, True, torch.float32) is not None:
            return x32
    if a.dtype == torch.float32:
        return x32.addmm_(a, w.t())
    return x32.add_(F.linear(a, w).float())


# ------------------------------------------------------------------------------------------------------- short convolution
def short_conv(inp, w, tail, rb, out):
    """Per-channel causal convolution over time + SiLU on the packed rows of ``inp`` ``[tokens, C]``; ``w`` ``[C, taps]``
    (last column = current token); ``tail`` ``[slots, taps-1, C]`` carries every sequence's last ``taps-1`` inputs and is
    updated.  A sequence with ``past == 0`` starts from zeros whatever its slot holds."""
    if _native(inp):
        count_launch(2)
        load_seq_ext().short_conv(inp, w, tail, rb.tok_seq, rb.seq_off, rb.slots, rb.past, out)
        return out
    taps = w.shape[1]
    wf = w.float()
    for b in range(rb.B):
        lo, n, slot = rb.offsets[b], rb.lens[b], rb.slot_list[b]
        prev = tail[slot].float() if rb.past_list[b] > 0 else torch.zeros(taps - 1, w.shape[0], device=inp.device)
        full = torch.cat([prev, inp[lo:lo + n].float()], 0)                    # [taps-1+n, C]
        win = full.unfold(0, taps, 1)                                           # [n, C, taps]
        acc = (win * wf).sum(-1)
        out[lo:lo + n] = F.silu(acc).to(out.dtype)
        if taps > 1:
            tail[slot] = full[full.shape[0] - (taps - 1):].to(tail.dtype)
    return out


# ------------------------------------------------------------------------------------------------------------- delta rule
def delta_scan(qkv, koff: int, voff: int, a, b, A_log, dt_bias, S, rb, kv_heads: int, chan: bool):
    """Gated delta rule over the packed rows.  ``qkv`` holds, per row, the convolved queries ``[kv_heads·D]`` at column 0,
    keys at ``koff`` and values ``[H·V]`` at ``voff``; ``a`` are the decay logits (``[tokens, H]``, or ``[tokens, H·D]``
    with ``chan``), ``b`` the write-strength logits ``[tokens, H]``; ``S`` ``[slots, H, D, V]`` fp32 is read (unless
    ``past == 0``) and left at the state after the last row.  Returns the read-outs ``[tokens, H·V]`` in fp32."""
    H, D, V = S.shape[1], S.shape[2], S.shape[3]
    out = torch.empty(qkv.shape[0], H * V, dtype=torch.float32, device=qkv.device)
    if _native(qkv):
        count_launch()
        load_seq_ext().delta_scan(qkv, koff, voff, a, b, A_log, dt_bias, S, rb.seq_off, rb.slots, rb.past, out, kv_heads, chan)
        return out
    rep = H // kv_heads
    rate = torch.exp(A_log.float())
    for bi in range(rb.B):
        lo, n, slot = rb.offsets[bi], rb.lens[bi], rb.slot_list[bi]
        st = S[slot].clone() if rb.past_list[bi] > 0 else torch.zeros(H, D, V, device=qkv.device)
        rows = qkv[lo:lo + n].float()
        q = rows[:, :kv_heads * D].view(n, kv_heads, D)
        k = rows[:, koff:koff + kv_heads * D].view(n, kv_heads, D)
        v = rows[:, voff:voff + H * V].view(n, H, V)
        q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / math.sqrt(D)
        k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)         # [n, H, D]
        beta = torch.sigmoid(b[lo:lo + n].float())
        al = a[lo:lo + n].float() + dt_bias.float()
        if chan:
            g = torch.exp(-rate[None, :, None] * F.softplus(al.view(n, H, D), threshold=20.0))
        else:
            g = torch.exp(-rate[None, :] * F.softplus(al, threshold=20.0))[:, :, None].expand(n, H, D)
        for t in range(n):
            st = st * g[t][:, :, None]
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", st, k[t]))
            st = st + k[t][:, :, None] * u[:, None, :]
            out[lo + t] = torch.einsum("hdv,hd->hv", st, q[t]).reshape(-1)
        S[slot] = st
    return out


def gated_rmsnorm(o, gate, w, eps: float, act: int, y, H: int, V: int):
    """``y[t, h, :] = o[t, h, :] / rms(o[t, h, :]) · w · act(gate[t, h, :])`` (``o`` fp32; ``act``: silu or sigmoid)."""
    if _native(o):
        count_launch()
        load_seq_ext().gated_rmsnorm(o, gate, w, float(eps), act, y, H, V)
        return y
    of = o.view(-1, H, V)
    g = gate.float().view(-1, H, V)
    g = F.silu(g) if act == GATE_SILU else torch.sigmoid(g)
    y.copy_((of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps) * w.float() * g).reshape(-1, H * V))
    return y


# ------------------------------------------------------------------------------------------- windowed attention on latents
def latent_gather(ring, cnew, rb, window: int):
    """Rows a windowed attention step needs, per sequence: the cached latents that the step's first query still sees
    (at most ``window - 1``), then the step's own.  Returns ``[rb.ext(window).rows, C]``."""
    ext = rb.ext(window)
    out = torch.empty(ext.rows, cnew.shape[1], dtype=cnew.dtype, device=cnew.device)
    if _native(cnew):
        count_launch()
        load_seq_ext().latent_gather(ring, cnew, ext.ext_seq, ext.ext_off, rb.seq_off, rb.slots, rb.past, out)
        return out
    L = ring.shape[1]
    for b in range(rb.B):
        lo, n, slot, past, np_, eo = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b], ext.npast[b], ext.offsets[b]
        for i in range(np_):
            out[eo + i] = ring[slot, (past - np_ + i) % L]
        out[eo + np_:eo + np_ + n] = cnew[lo:lo + n]
    return out


def latent_write(ring, cnew, rb):
    """Store the step's latents: position p of a sequence goes to ``ring[slot, p % ring_len]``."""
    if _native(cnew):
        count_launch()
        load_seq_ext().latent_write(ring, cnew, rb.tok_seq, rb.seq_off, rb.slots, rb.past)
        return
    L = ring.shape[1]
    for b in range(rb.B):
        lo, n, slot, past = rb.offsets[b], rb.lens[b], rb.slot_list[b], rb.past_list[b]
        for t in range(max(0, n - L), n):
            ring[slot, (past + t) % L] = cnew[lo + t]


def window_attention(q, kv, gate, rb, y, H: int, D: int, V: int, window: int, scale: float, mma: bool = True):
    """Softmax attention of every packed query over the ``window`` rows of ``kv`` (keys ``[H·D]`` then values ``[H·V]`` per
    row, laid out as :func:`latent_gather` orders them) that end at its own row; head ``h`` of the result is multiplied by
    ``sigmoid(gate[t, h])`` when a gate is given.  Writes ``y`` ``[tokens, H·V]``.  bf16 inputs with head sizes the tensor-core
    kernel is built for (32 / 64 / 128) take it; ``mma=False`` keeps them on the generic kernel (fp32 inputs always are)."""
    ext = rb.ext(window)
    if _native(q):
        count_launch()
        tiles = rb.query_tiles(64) if (q.dtype == torch.bfloat16 and mma) else (None, None)
        load_seq_ext().window_attention(q, kv, gate, rb.tok_seq, rb.seq_off, ext.ext_off, tiles[0], tiles[1], y, H, D, V, window,
                                        float(scale))
        return y
    for b in range(rb.B):
        lo, n, np_, eo = rb.offsets[b], rb.lens[b], ext.npast[b], ext.offsets[b]
        rows = kv[eo:eo + np_ + n].float()
        k = rows[:, :H * D].view(-1, H, D)
        v = rows[:, H * D:].view(-1, H, V)
        qq = q[lo:lo + n].float().view(n, H, D)
        s = torch.einsum("thd,jhd->htj", qq, k) * scale
        ti = torch.arange(n, device=q.device)[:, None] + np_
        ji = torch.arange(np_ + n, device=q.device)[None, :]
        s = s.masked_fill(~((ji <= ti) & (ti - ji < window)), float("-inf"))
        o = torch.einsum("htj,jhv->thv", torch.softmax(s, -1), v)
        if gate is not None:
            o = o * torch.sigmoid(gate[lo:lo + n].float())[:, :, None]
        y[lo:lo + n] = o.reshape(n, H * V).to(y.dtype)
    return y


def latent_decode(qa, ring, cnew, rb, window: int, scale: float):
    """Single-token steps in the absorbed form: ``qa`` ``[B, H, C]`` fp32 are the queries already multiplied by the key
    up-projection, so scores and the weighted sum run on the latents themselves (the ring for older positions, ``cnew`` for
    the current one).  Returns the softmax-weighted latents ``[B, H, C]`` fp32."""
    out = torch.empty_like(qa)
    if _native(qa):
        count_launch()
        load_seq_ext().latent_decode(qa, ring, cnew, rb.slots, rb.past, out, window, float(scale))
        return out
    L = ring.shape[1]
    for b in range(rb.B):
        p, slot = rb.past_list[b], rb.slot_list[b]
        lat = [ring[slot, j % L].float() for j in range(max(0, p - window + 1), p)] + [cnew[b].float()]
        lat = torch.stack(lat)                                                    # [visible, C]
        pr = torch.softmax(torch.einsum("hc,jc->hj", qa[b], lat) * scale, -1)
        out[b] = pr @ lat
    return out


def head_gate(x, gate, y, H: int, V: int):
    """``y[t, h·V + v] = x[t, h, v] · sigmoid(gate[t, h])`` (``x`` fp32 ``[tokens, H, V]``)."""
    if _native(x):
        count_launch()
        load_seq_ext().head_gate(x, gate, y, H, V)
        return y
    o = x.view(-1, H, V)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())[:, :, None]
    y.copy_(o.reshape(-1, H * V))
    return y


# ------------------------------------------------------------------------------------------------------------ projections
def linear(a, w):
    """``a @ wᵀ`` for a row-major view ``a`` ``[rows, K]`` (its rows may be a column slice of a wider matrix): the tcgen05
    GEMM reads the slice in place through its row stride; shapes it does not take, fp32 operands and CPU tensors go to the
    vendor / PyTorch product."""
    from . import load_ext, use_native

    if (a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and use_native(a) and a.dim() == 2
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.shape[1] % 8 == 0 and w.is_contiguous()
            and w.shape[0] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.shape[0] > 0):
        y = _tcgen05_gemm(a, w, None, False, torch.bfloat16)
        if y is not None:
            return y
    return F.linear(a, w)


_GEMM_REFUSED = set()


def _tcgen05_gemm(a, w, out, accumulate, out_dtype):
    """The framework's GEMM; a shape it refuses (the launcher returns an error code before anything runs) is remembered and
    sent to the vendor product from then on — ``None`` tells the caller to do so."""
    from . import load_ext

    key = (a.shape[0] > 1, a.shape[1], w.shape[0], a.stride(0), accumulate)
    if key in _GEMM_REFUSED:
        return None
    try:
        y = load_ext().gemm(a, w, 0, None, out, accumulate, out_dtype)
    except RuntimeError as e:
        if "failed with code -" not in str(e):          # a CUDA error, not a refusal by the launcher's shape checks
            raise
        _GEMM_REFUSED.add(key)
        return None
    count_launch()
    return y


def fuse_rows(named, align: int = 8):
    """Stack ``[(name, W [n_i, K]), …]`` into one ``[Σ pad(n_i), K]`` matrix (every segment starts on a multiple of ``align``
    rows, padding rows are zero) so that several projections of the same input are ONE product; returns the matrix and
    ``{name: (first column of the product, n_i)}``."""
    parts, where, at = [], {}, 0
    for name, w in named:
        n = w.shape[0]
        where[name] = (at, n)
        parts.append(w)
        pad = (-n) % align
        if pad:
            parts.append(w.new_zeros(pad, w.shape[1]))
        at += n + pad
    return torch.cat(parts, 0).contiguous(), where


def fuse_cols(named, align: int = 8):
    """Concatenate ``[(name, W [N, k_i]), …]`` along the input dimension (segments padded with zero columns to a multiple of
    ``align``): ``Σ_i W_i y_i`` becomes one product on the concatenated inputs.  Returns the matrix and ``{name: (first
    column, k_i)}``."""
    parts, where, at = [], {}, 0
    for name, w in named:
        k = w.shape[1]
        where[name] = (at, k)
        parts.append(w)
        pad = (-k) % align
        if pad:
            parts.append(w.new_zeros(w.shape[0], pad))
        at += k + pad
    return torch.cat(parts, 1).contiguous(), where
