"""Salizen checkpoints (``config.json`` + ``model.safetensors``) → :class:`libai_b200.models.SalizenForCausalLM`.

``config.json``: ``vocab``, ``width``, ``streams``, ``norm.eps``, ``embedding`` (``scale``, ``bigram``: ``buckets``, ``mul_prev``,
``mul_cur``) and ``layers`` (per block ``type``, ``mixer`` sizes and constants, ``mlp``: ``{kind: dense, ff}``,
``{kind: moe, expert: {ff}, router: {experts, top}}`` or null).  Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and
per block ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.<name>`` (a parallel mixer: ``l<i>.mix.left.<name>`` and
``l<i>.mix.right.<name>``; the bias of the decay logits is ``a2.b``), ``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router`` (+ ``.b``)
and ``l<i>.mlp.e<j>.gate|up|down``.  Linear weights are ``[out, in]``; a dense feed-forward's ``gate`` and ``up`` are stacked into
``gate_up`` ``[2·ff, width]``, the experts' matrices into ``gate_up`` ``[E, 2·ff, width]`` and ``down`` ``[E, width, ff]``.  The inner
size of a decay's low-rank pair is not in the configuration; it is read off the tensor shapes.
"""
import collections
import re

import torch

from .base_loader import ModelLoaderHuggerFace

_TOP = {"embed": "model.embed", "bigram": "model.bigram", "final.norm": "model.final_norm.weight", "head": "head"}
_HC = {"in": "inw", "out": "outw", "mix": "mix"}


class SalizenLoader(ModelLoaderHuggerFace):
    def _load_config_from_json(self, config_file):
        cfg = self._read_config_json()
        for key in ("vocab", "width", "streams", "layers", "norm", "embedding"):
            if key in cfg:
                self._update_cfg(key, cfg[key])
        for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if cfg.get(key) is not None:
                self._update_cfg(key, cfg[key])

    def _convert_state_dict(self, sd, cfg):
        for i, lc in enumerate(cfg["layers"]):
            if lc["type"] == "parallel" and f"l{i}.mix.right.a1" in sd:
                lc["mixer"]["right"]["decay_rank"] = int(sd[f"l{i}.mix.right.a1"].shape[0])
        out = collections.OrderedDict()
        experts = collections.defaultdict(dict)                # (block, matrix) -> {expert: tensor}
        dense = collections.defaultdict(dict)                  # block -> {gate | up: tensor}
        for name, t in sd.items():
            if name in _TOP:
                out[_TOP[name]] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(norm1|norm2)", name)
            if m:
                out[f"model.layers.{m.group(1)}.{m.group(2)}.weight"] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(hc1|hc2)\.(in|out|mix)", name)
            if m:
                out[f"model.layers.{m.group(1)}.{m.group(2)}.{_HC[m.group(3)]}"] = t
                continue
            m = re.fullmatch(r"l(\d+)\.mlp\.e(\d+)\.(gate|up|down)", name)
            if m:
                experts[(m.group(1), m.group(3))][int(m.group(2))] = t
                continue
            m = re.fullmatch(r"l(\d+)\.mlp\.(gate|up)", name)
            if m:
                dense[m.group(1)][m.group(2)] = t
                continue
            m = re.fullmatch(r"l(\d+)\.mlp\.(down|router|router\.b)", name)
            if m:
                out[f"model.layers.{m.group(1)}.mlp.{m.group(2).replace('.', '_')}"] = t
                continue
            m = re.fullmatch(r"l(\d+)\.mix\.((?:left\.|right\.)?)(.+)", name)
            if m:
                out[f"model.layers.{m.group(1)}.mix.{m.group(2)}{m.group(3).replace('.', '_')}"] = t
                continue
            out[name] = t                                      # reported as unexpected by the base loader
        for i, parts in dense.items():
            if sorted(parts) != ["gate", "up"]:
                raise ValueError(f"block {i}: a dense feed-forward needs both gate and up")
            out[f"model.layers.{i}.mlp.gate_up"] = torch.cat([parts["gate"], parts["up"]], 0)
        for i in sorted({i for i, _ in experts}, key=int):
            gate, up, down = experts[(i, "gate")], experts[(i, "up")], experts[(i, "down")]
            order = sorted(gate)
            if order != list(range(len(order))) or sorted(up) != order or sorted(down) != order:
                raise ValueError(f"block {i}: the experts' tensors are not e0 … e{len(order) - 1} with gate, up and down each")
            out[f"model.layers.{i}.mlp.gate_up"] = torch.stack([torch.cat([gate[e], up[e]], 0) for e in order])
            out[f"model.layers.{i}.mlp.down"] = torch.stack([down[e] for e in order])
        return out
