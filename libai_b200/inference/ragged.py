"""Ragged step descriptor: which sequences a step carries, how many new tokens each brings, where their state lives.

The generation path of the stateful models works on packed rows (no padding): sequence ``b`` owns rows
``offsets[b] … offsets[b] + lens[b] - 1`` of every activation matrix of the step, its state sits in slot ``slots[b]`` of the
:class:`~libai_b200.inference.state_cache.SequenceStateCache` and already covers ``past[b]`` tokens.  The descriptor is built
on the host and shipped to the device as ONE int32 tensor; the kernels index it directly.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch


class WindowExt:
    """Row layout of the keys of a windowed attention step: per sequence the ``npast[b] = min(past[b], window - 1)`` cached
    positions its first query still sees, then its new tokens."""

    def __init__(self, rb: "RaggedBatch", window: int):
        self.npast = [min(p, window - 1) for p in rb.past_list]
        lens = [a + n for a, n in zip(self.npast, rb.lens)]
        self.offsets = [0]
        for n in lens:
            self.offsets.append(self.offsets[-1] + n)
        self.rows = self.offsets[-1]
        seq = [b for b, n in enumerate(lens) for _ in range(n)]
        packed = torch.tensor(self.offsets + seq, dtype=torch.int32).to(rb.device, non_blocking=True)
        self.ext_off, self.ext_seq = packed[: rb.B + 1], packed[rb.B + 1:]


def mask_floor(position: int, window: int, chunk: int) -> int:
    """First position of the contiguous range that the query at ``position`` sees under a chunk mask (``chunk > 0``: its own
    chunk, counted from position 0) or a sliding window (``window > 0``); 0 when neither bounds it."""
    if chunk > 0:
        return (position // chunk) * chunk
    if window > 0:
        return max(0, position - window + 1)
    return 0


class KvExt:
    """Row layout of the keys / values of a prompt step over ring caches, shared by every layer that reads the same cache
    (each with its own mask ``(window, chunk, keep)``): per sequence the kept-first positions that are older than the
    contiguous part (``nsink`` rows, positions 0 …), the cached positions ``cstart … past − 1``, then the step's own rows.
    ``cstart`` is the earliest position the step's first query sees under any of the masks."""

    def __init__(self, rb: "RaggedBatch", masks):
        self.cstart_list = [min(mask_floor(p, w, c) for w, c, _ in masks) for p in rb.past_list]
        keep = max([k for w, c, k in masks if c <= 0] + [0])
        self.nsink_list = [min(keep, cs) for cs in self.cstart_list]
        lens = [ns + (p - cs) + n for ns, cs, p, n in zip(self.nsink_list, self.cstart_list, rb.past_list, rb.lens)]
        self.offsets = [0]
        for n in lens:
            self.offsets.append(self.offsets[-1] + n)
        self.rows = self.offsets[-1]
        self.cached = any(ns + p - cs > 0 for ns, cs, p in zip(self.nsink_list, self.cstart_list, rb.past_list))
        seq = [b for b, n in enumerate(lens) for _ in range(n)] if self.cached else []
        packed = torch.tensor(self.offsets + self.nsink_list + self.cstart_list + seq, dtype=torch.int32)
        packed = packed.to(rb.device, non_blocking=True)
        B = rb.B
        self.ext_off, self.nsink, self.cstart = packed[: B + 1], packed[B + 1: 2 * B + 1], packed[2 * B + 1: 3 * B + 1]
        self.ext_seq = packed[3 * B + 1:]


class RaggedBatch:
    def __init__(self, lens: Sequence[int], slots: Sequence[int], past: Sequence[int], device):
        assert len(lens) == len(slots) == len(past) and all(n > 0 for n in lens)
        self.B, self.device = len(lens), torch.device(device)
        self.lens, self.slot_list, self.past_list = list(lens), list(slots), list(past)
        self.offsets: List[int] = [0]
        for n in self.lens:
            self.offsets.append(self.offsets[-1] + n)
        self.tokens = self.offsets[-1]
        self.single = all(n == 1 for n in self.lens)          # every sequence goes on by one token
        tok_seq = [b for b, n in enumerate(self.lens) for _ in range(n)]
        packed = torch.tensor(self.offsets + self.slot_list + self.past_list + tok_seq, dtype=torch.int32)
        packed = packed.to(self.device, non_blocking=True)
        B = self.B
        self.seq_off, self.slots, self.past = packed[: B + 1], packed[B + 1: 2 * B + 1], packed[2 * B + 1: 3 * B + 1]
        self.tok_seq = packed[3 * B + 1:]
        self._ext: Dict[int, WindowExt] = {}
        self._kv_ext: Dict[tuple, KvExt] = {}
        self._tiles: Dict[int, tuple] = {}

    def ext(self, window: int) -> WindowExt:
        if window not in self._ext:
            self._ext[window] = WindowExt(self, window)
        return self._ext[window]

    def kv_ext(self, masks) -> KvExt:
        """Key / value row layout of this step for a cache read under the masks ``((window, chunk, keep), …)``."""
        key = tuple(sorted(set(tuple(m) for m in masks)))
        if key not in self._kv_ext:
            self._kv_ext[key] = KvExt(self, key)
        return self._kv_ext[key]

    def query_tiles(self, size: int):
        """Tiles of ``size`` consecutive new tokens of one sequence: (sequence of every tile, its first token) on the device."""
        if size not in self._tiles:
            seq = [b for b, n in enumerate(self.lens) for _ in range(0, n, size)]
            start = [t for n in self.lens for t in range(0, n, size)]
            packed = torch.tensor(seq + start, dtype=torch.int32).to(self.device, non_blocking=True)
            self._tiles[size] = (packed[: len(seq)], packed[len(seq):])
        return self._tiles[size]

    def last_rows(self) -> List[int]:
        """Packed row of every sequence's last new token."""
        return [self.offsets[b + 1] - 1 for b in range(self.B)]
