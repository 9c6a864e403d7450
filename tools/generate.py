"""Generate from a checkpoint folder (``config.json`` + weights) on token ids.

    python tools/generate.py --model DIR --prompts "5 17 3;9 9 12 40" --max-new-tokens 16 [--dtype float32] [--do-sample …]

The model class and loader come from ``config.json`` (``libai_b200.models.utils.model_loader.auto``).  Models with per-sequence
state (Bumodra, Nefelorn, Salizen) run through ``RequestScheduler.generate``: one ragged step for all prompts, then one token per live request;
the others through ``Generator.generate`` on a left-padded batch.  Prints one line of generated ids per prompt.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

import torch  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompts", required=True, help="token ids separated by blanks, prompts separated by ';'")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--device", default=None)
    ap.add_argument("--do-sample", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--eos-token-id", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    if device.startswith("cuda"):
        from libai_b200.models.utils.model_loader.auto import native_libs_of
        from libai_b200.ops import build

        build.build(only=native_libs_of(a.model, dtype) + ["_C"])
    from libai_b200.models.utils.model_loader.auto import load_pretrained

    model = load_pretrained(a.model, dtype=dtype, device=device)
    prompts = [[int(t) for t in p.split()] for p in a.prompts.split(";") if p.strip()]
    torch.manual_seed(a.seed)
    if hasattr(model, "step"):
        from libai_b200.inference.scheduler import RequestScheduler

        out = RequestScheduler(model).generate(prompts, a.max_new_tokens, eos_token_id=a.eos_token_id, do_sample=a.do_sample,
                                               temperature=a.temperature, top_k=a.top_k, top_p=a.top_p)
    else:
        pad = model._gcfg("pad_token_id") or 0
        width = max(len(p) for p in prompts)
        ids = torch.tensor([[pad] * (width - len(p)) + p for p in prompts])
        full = model.generate(ids, max_new_tokens=a.max_new_tokens, do_sample=a.do_sample, temperature=a.temperature,
                              top_k=a.top_k or None, top_p=a.top_p, eos_token_id=a.eos_token_id, pad_token_id=pad)
        out = [row[width:].tolist() for row in full]
    for row in out:
        print(" ".join(str(t) for t in row))
    return out


if __name__ == "__main__":
    main()
