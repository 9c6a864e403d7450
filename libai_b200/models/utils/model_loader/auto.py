"""Pick the model class and its loader from a checkpoint folder's ``config.json``.

``load_pretrained(path)`` reads ``architecture`` / ``architectures[0]`` / ``model_type``, looks the name up in
:data:`ARCHITECTURES` and returns the loaded model in eval mode on the requested device and dtype."""
import json
import os

import torch

from libai_b200.config import DictConfig
from libai_b200.layers._param import param_defaults


def _llama():
    from libai_b200.models import LlamaForCausalLM
    from .llama_loader import LlamaLoaderHuggerFace

    defaults = dict(hidden_layers=1, vocab_size=1, hidden_size=8, intermediate_size=8, num_attention_heads=1,
                    max_position_embeddings=2048, rms_norm_eps=1e-5, initializer_range=0.02,
                    use_scaled_init_for_output_weights=True, scale_mask_softmax_fusion=False, amp_enabled=False)
    return LlamaForCausalLM, LlamaLoaderHuggerFace, defaults


def _bumodra():
    from libai_b200.models import BumodraForCausalLM
    from .bumodra_loader import BumodraLoader

    return BumodraForCausalLM, BumodraLoader, {}


def _nefelorn():
    from libai_b200.models import NefelornForCausalLM
    from .nefelorn_loader import NefelornLoader

    return NefelornForCausalLM, NefelornLoader, {}


def _salizen():
    from libai_b200.models import SalizenForCausalLM
    from .salizen_loader import SalizenLoader

    return SalizenForCausalLM, SalizenLoader, {}


def _zubarax():
    from libai_b200.models import ZubaraxForCausalLM
    from .zubarax_loader import ZubaraxLoader

    return ZubaraxForCausalLM, ZubaraxLoader, {}


ARCHITECTURES = {
    "bumodra": _bumodra,
    "nefelorn": _nefelorn,
    "salizen": _salizen,
    "zubarax": _zubarax,
    "llama": _llama, "llamaforcausallm": _llama,
}


# native libraries (``libai_b200.ops.build``) that a model's generation path launches besides the GEMM library ``_C``
NATIVE_LIBS = {"bumodra": ["_C_seq"], "nefelorn": ["_C_kv"], "salizen": ["_C_kv", "_C_lin"],
               "zubarax": ["_C_kv", "_C_lin"]}


def native_libs_of(path: str, dtype=torch.bfloat16):
    """Names of the in-tree libraries that serving the checkpoint at ``path`` in ``dtype`` needs: the model's own kernels, and
    the tcgen05 GEMM library only where bf16 products run on it."""
    return NATIVE_LIBS.get(architecture_of(path), []) + (["_C"] if dtype == torch.bfloat16 else [])


def architecture_of(path: str) -> str:
    with open(os.path.join(path, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    name = cfg.get("architecture") or (cfg.get("architectures") or [None])[0] or cfg.get("model_type")
    if name is None or str(name).lower() not in ARCHITECTURES:
        raise ValueError(f"config.json of {path} names no known architecture ({name!r}); known: {sorted(ARCHITECTURES)}")
    return str(name).lower()


def load_pretrained(path: str, dtype=torch.bfloat16, device=None, **overrides):
    model_cls, loader_cls, defaults = ARCHITECTURES[architecture_of(path)]()
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    cfg = DictConfig({**defaults, **overrides})
    with param_defaults(dtype=dtype, device=device):
        model = loader_cls(model_cls, cfg, path).load()
    return model.eval()
