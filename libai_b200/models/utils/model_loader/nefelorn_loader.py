"""Nefelorn checkpoints (``config.json`` + ``model.safetensors``) → :class:`libai_b200.models.NefelornForCausalLM`.

``config.json``: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``logit_softcap`` and ``layers`` (per block ``type``,
``mixer`` sizes with ``mask``, ``rot``, ``scale`` and optionally ``kv_from``, and ``mlp``: ``{kind: dense, ff}``,
``{kind: moe, expert: {ff}, router: {experts, top, scale}}`` or null).  Tensor names: ``embed``, ``final.norm`` (+ ``.b``,
``.alpha``), ``head`` and per block ``l<i>.norm1|norm1b|norm2|norm2b`` (+ ``.b``, ``.alpha``), ``l<i>.mix.q|k|v|g|o``,
``l<i>.mix.q.norm|k.norm``, ``l<i>.mlp.up|down`` or ``l<i>.mlp.router`` and ``l<i>.mlp.e<j>.gate|up|down``.  Linear weights
are ``[out, in]``; the experts' matrices are stacked into ``gate_up`` ``[E, 2·ff, width]`` and ``down`` ``[E, width, ff]``.
"""
import collections
import re

import torch

from .base_loader import ModelLoaderHuggerFace

_NORM = {None: "weight", "b": "bias", "alpha": "alpha"}


class NefelornLoader(ModelLoaderHuggerFace):
    def _load_config_from_json(self, config_file):
        cfg = self._read_config_json()
        for key in ("vocab", "width", "layers", "norm", "embedding", "logit_softcap"):
            if key in cfg:
                self._update_cfg(key, cfg[key])
        for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if cfg.get(key) is not None:
                self._update_cfg(key, cfg[key])

    def _convert_state_dict(self, sd, cfg):
        out = collections.OrderedDict()
        experts = collections.defaultdict(dict)                # (block, matrix) -> {expert: tensor}
        for name, t in sd.items():
            if name in ("embed", "head"):
                out["model.embed" if name == "embed" else "head"] = t
                continue
            m = re.fullmatch(r"final\.norm(?:\.(b|alpha))?", name)
            if m:
                out[f"model.final_norm.{_NORM[m.group(1)]}"] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(norm1b|norm2b|norm1|norm2)(?:\.(b|alpha))?", name)
            if m:
                out[f"model.layers.{m.group(1)}.{m.group(2)}.{_NORM[m.group(3)]}"] = t
                continue
            m = re.fullmatch(r"l(\d+)\.mlp\.e(\d+)\.(gate|up|down)", name)
            if m:
                experts[(m.group(1), m.group(3))][int(m.group(2))] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(mix|mlp)\.(.+)", name)
            if m:
                out[f"model.layers.{m.group(1)}.{m.group(2)}.{m.group(3).replace('.', '_')}"] = t
                continue
            out[name] = t                                      # reported as unexpected by the base loader
        for i in sorted({i for i, _ in experts}, key=int):
            gate, up, down = experts[(i, "gate")], experts[(i, "up")], experts[(i, "down")]
            order = sorted(gate)
            if order != list(range(len(order))) or sorted(up) != order or sorted(down) != order:
                raise ValueError(f"block {i}: the experts' tensors are not e0 … e{len(order) - 1} with gate, up and down each")
            out[f"model.layers.{i}.mlp.gate_up"] = torch.stack([torch.cat([gate[e], up[e]], 0) for e in order])
            out[f"model.layers.{i}.mlp.down"] = torch.stack([down[e] for e in order])
        return out
