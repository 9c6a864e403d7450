"""A small Zubarax causal LM: post-norm blocks whose mixer runs paged softmax attention (short convolutions, mixed heads, a
learned sink) beside an HGRN2 recurrence, mixture-of-experts feed-forwards with a shared expert; the last two entries run the
first two blocks again with a state of their own.  Checkpoint folders carry their own ``config.json``; this record is for
random-init runs."""
from libai_b200.config import DictConfig, LazyCall
from libai_b200.models import ZubaraxForCausalLM


def _moe(ff, experts=8, top=2, limit=7.0):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top), shared=dict(ff=2 * ff, limit=limit))


def _parallel(mlp=None, weights_of=None):
    left = dict(heads=8, kv_heads=2, dim=64, vdim=64, conv=4, scale=0.125, rot=dict(dims=32, base=500000.0))
    right = dict(heads=4, dim=64, vdim=128)
    out = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0), mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


cfg = DictConfig(
    dict(
        vocab=32000, width=512, norm=dict(eps=1e-6), postln_alpha=2.0, embedding=dict(scale=22.6),
        layers=[_parallel(mlp=_moe(512)), _parallel(mlp=_moe(512)), _parallel(mlp=_moe(512), weights_of=0), _parallel(mlp=_moe(512), weights_of=1)],
        initializer_range=0.02, kv_page_size=64,
        # generation defaults
        is_encoder_decoder=False, max_length=256, do_sample=False, num_beams=1, temperature=1.0, top_k=50, top_p=1.0,
        use_cache=True, bos_token_id=1, eos_token_id=2, pad_token_id=0,
    )
)

model = LazyCall(ZubaraxForCausalLM)(cfg=cfg)
