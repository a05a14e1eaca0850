"""Bumodra checkpoints (``config.json`` + ``model.safetensors``) → :class:`libai_b200.models.BumodraForCausalLM`.

``config.json``: ``vocab``, ``width``, ``norm.eps``, ``layers`` (per block ``type``, ``mixer`` sizes, ``mlp`` or null) and
``loop`` (``start``, ``stop``, ``times``; may be absent).  Tensor names: ``embed``, ``embed.norm``, ``loop.in``,
``final.norm``, ``head`` and per block ``l<i>.norm1``, ``l<i>.mix.<name>`` (a convolution is ``<name>.conv``, a latent's norm
``<name>.norm``), ``l<i>.mlp.up|down``.  Linear weights are ``[out, in]``.  The ranks of the low-rank decay / gate pairs of a
``channel_delta`` mixer are not in the configuration; they are read off the tensor shapes.
"""
import collections
import re

from .base_loader import ModelLoaderHuggerFace

_TOP = {"embed": "model.embed", "embed.norm": "model.embed_norm.weight", "loop.in": "model.loop_in",
        "final.norm": "model.final_norm.weight", "head": "head"}


class BumodraLoader(ModelLoaderHuggerFace):
    def _load_config_from_json(self, config_file):
        cfg = self._read_config_json()
        for key in ("vocab", "width", "layers", "loop", "norm"):
            if key in cfg:
                self._update_cfg(key, cfg[key])
        for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if cfg.get(key) is not None:
                self._update_cfg(key, cfg[key])

    def _convert_state_dict(self, sd, cfg):
        layers = cfg["layers"]
        for i, lc in enumerate(layers):
            if lc["type"] == "channel_delta":
                lc["mixer"]["decay_rank"] = int(sd[f"l{i}.mix.a1"].shape[0])
                lc["mixer"]["gate_rank"] = int(sd[f"l{i}.mix.g1"].shape[0])
        out = collections.OrderedDict()
        for name, t in sd.items():
            if name in _TOP:
                out[_TOP[name]] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(norm1|mix|mlp)(?:\.(.+))?", name)
            if m is None:
                out[name] = t                                  # reported as unexpected by the base loader
                continue
            i, part, rest = m.group(1), m.group(2), m.group(3)
            if part == "norm1":
                out[f"model.layers.{i}.norm1.weight"] = t
            else:
                out[f"model.layers.{i}.{part}.{rest.replace('.', '_')}"] = t
        return out
