"""Zubarax checkpoints (``config.json`` + ``model.safetensors``) → :class:`libai_b200.models.ZubaraxForCausalLM`.

``config.json``: ``vocab``, ``width``, ``norm.eps``, ``postln_alpha``, ``embedding.scale`` and ``layers`` (per entry ``type``, ``mixer`` sizes
and constants, ``mlp``: ``{kind: moe, expert: {ff, limit}, router: {experts, top}, shared: {ff, limit}}`` or null, and optionally
``weights_of: j`` for an entry that runs entry j's tensors).  Tensor names: ``embed``, ``final.norm`` and per entry that owns
tensors ``l<i>.norm1|norm2``, ``l<i>.mix.left.q|k|v|o``, ``l<i>.mix.left.q|k|v.conv``, ``l<i>.mix.left.q|k.norm``, ``l<i>.mix.left.talk|sink``,
``l<i>.mix.right.q|f|v|o``, ``l<i>.mix.right.f.b|lower|norm``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down`` and
``l<i>.mlp.shared.gate|up|down``.  Linear weights are ``[out, in]``; the experts' matrices are stacked into ``gate_up``
``[E, 2·ff, width]`` and ``down`` ``[E, width, ff]``, the shared expert's ``gate`` and ``up`` into ``gate_up`` ``[2·ff, width]``.  The model
keeps one block per entry that owns tensors; entry i's tensors go to block ``owners.index(i)``.
"""
import collections
import re

import torch

from .base_loader import ModelLoaderHuggerFace

_TOP = {"embed": "model.embed", "final.norm": "model.final_norm.weight"}


class ZubaraxLoader(ModelLoaderHuggerFace):
    def _load_config_from_json(self, config_file):
        cfg = self._read_config_json()
        for key in ("vocab", "width", "layers", "norm", "embedding", "postln_alpha", "kv_page_size"):
            if key in cfg:
                self._update_cfg(key, cfg[key])
        for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if cfg.get(key) is not None:
                self._update_cfg(key, cfg[key])

    def _convert_state_dict(self, sd, cfg):
        owners = [i for i, lc in enumerate(cfg["layers"]) if lc.get("weights_of") is None]
        block = {str(i): k for k, i in enumerate(owners)}
        # an entry without a feed-forward whose second norm is in the checkpoint applies it to alpha · x alone
        bare = [i for i in owners if not cfg["layers"][i].get("mlp") and f"l{i}.norm2" in sd]
        if bare:
            layers = [dict(lc) for lc in cfg["layers"]]
            for i in bare:
                layers[i]["bare_norm2"] = True
            self._update_cfg("layers", layers)
        out = collections.OrderedDict()
        experts = collections.defaultdict(dict)                # (block, matrix) -> {expert: tensor}
        shared = collections.defaultdict(dict)                 # block -> {gate | up: tensor}
        for name, t in sd.items():
            if name in _TOP:
                out[_TOP[name]] = t
                continue
            m = re.fullmatch(r"l(\d+)\.(.+)", name)
            if not m or m.group(1) not in block:
                out[name] = t                                  # reported as unexpected by the base loader
                continue
            k, rest = block[m.group(1)], m.group(2)
            pre = f"model.layers.{k}."
            if rest in ("norm1", "norm2"):
                out[pre + rest + ".weight"] = t
                continue
            m = re.fullmatch(r"mlp\.e(\d+)\.(gate|up|down)", rest)
            if m:
                experts[(k, m.group(2))][int(m.group(1))] = t
                continue
            m = re.fullmatch(r"mlp\.shared\.(gate|up)", rest)
            if m:
                shared[k][m.group(1)] = t
                continue
            if rest == "mlp.shared.down":
                out[pre + "shared.down"] = t
                continue
            if rest == "mlp.router":
                out[pre + "mlp.router"] = t
                continue
            m = re.fullmatch(r"mix\.(left|right)\.(.+)", rest)
            if m:
                out[f"{pre}mix.{m.group(1)}.{m.group(2).replace('.', '_')}"] = t
                continue
            out[name] = t
        for k, parts in shared.items():
            if sorted(parts) != ["gate", "up"]:
                raise ValueError(f"block {k}: a shared expert needs both gate and up")
            out[f"model.layers.{k}.shared.gate_up"] = torch.cat([parts["gate"], parts["up"]], 0)
        for k in sorted({k for k, _ in experts}):
            gate, up, down = experts[(k, "gate")], experts[(k, "up")], experts[(k, "down")]
            order = sorted(gate)
            if order != list(range(len(order))) or sorted(up) != order or sorted(down) != order:
                raise ValueError(f"block {k}: the experts' tensors are not e0 … e{len(order) - 1} with gate, up and down each")
            out[f"model.layers.{k}.mlp.gate_up"] = torch.stack([torch.cat([gate[e], up[e]], 0) for e in order])
            out[f"model.layers.{k}.mlp.down"] = torch.stack([down[e] for e in order])
        return out

    def _load(self, model, state_dict):
        """Every parameter of the model must come from the checkpoint: a tensor that is missing would otherwise stay at its
        random initial value."""
        missing = sorted(set(model.state_dict().keys()) - set(state_dict.keys()))
        if missing:
            raise RuntimeError(f"the checkpoint at {self.pretrained_model_path} lacks tensors for: {missing}")
        return super()._load(model, state_dict)
