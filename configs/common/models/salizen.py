"""A small Salizen causal LM: two residual streams, a parallel block (sink-softmax window attention beside gated linear attention),
a retention block and two lightning blocks, dense and mixture-of-experts feed-forwards.  Checkpoint folders carry their own
``config.json``; this record is for random-init runs."""
from libai_b200.config import DictConfig, LazyCall
from libai_b200.models import SalizenForCausalLM


def _moe(ff, experts=8, top=2):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def _parallel(mlp=None):
    left = dict(heads=8, kv_heads=2, dim=64, vdim=64, mask=dict(size=512), scale=0.125, softcap=30.0,
                rot=dict(dims=32, base=1000000.0, scaling=dict(factor=8.0, original=8192, low=1.0, high=4.0)))
    right = dict(heads=4, dim=64, vdim=128, tau=8.0, decay_rank=16)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0), mlp=mlp)


def _retention(mlp=None):
    return dict(type="retention", mlp=mlp,
                mixer=dict(heads=8, dim=64, vdim=64, decay=[1.0 - 2.0 ** (-5 - i) for i in range(8)], rot=dict(dims=64, base=10000.0)))


def _lightning(mlp=None):
    return dict(type="lightning", mlp=mlp, mixer=dict(heads=8, dim=64, vdim=64, decay=[1.0 - 2.0 ** (-3 - i) for i in range(8)]))


cfg = DictConfig(
    dict(
        vocab=32000, width=512, streams=2, norm=dict(eps=1e-6),
        embedding=dict(scale=22.6, bigram=dict(buckets=65521, mul_prev=31, mul_cur=13)),
        layers=[_parallel(mlp=dict(kind="dense", ff=1408)), _retention(mlp=_moe(512)), _lightning(mlp=dict(kind="dense", ff=1408)),
                _lightning(mlp=_moe(512))],
        initializer_range=0.02,
        # generation defaults
        is_encoder_decoder=False, max_length=256, do_sample=False, num_beams=1, temperature=1.0, top_k=50, top_p=1.0,
        use_cache=True, bos_token_id=1, eos_token_id=2, pad_token_id=0,
    )
)

model = LazyCall(SalizenForCausalLM)(cfg=cfg)
