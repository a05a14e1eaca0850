"""A small Nefelorn causal LM: chunked attention blocks with a whole-projection query/key norm and blended rotary frequencies (the
third reads the first one's keys), sliding-window blocks that keep the first tokens, dense and mixture-of-experts feed-forwards.
Checkpoint folders carry their own ``config.json``; this record is for random-init runs."""
from libai_b200.config import DictConfig, LazyCall
from libai_b200.models import NefelornForCausalLM


def _moe(ff, experts=8, top=2):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=1.0))


def _chunked(kv_from=None, mlp=None):
    m = dict(heads=8, kv_heads=2, dim=64, vdim=64, mask=dict(size=256), scale=0.125,
             rot=dict(dims=64, base=500000.0, scaling=dict(factor=4.0, original=4096, fast=24.0, slow=2.0)))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def _windowed(mlp=None):
    return dict(type="attention_2", mlp=mlp,
                mixer=dict(heads=8, kv_heads=2, dim=64, vdim=64, mask=dict(size=512, keep_first=8), scale=0.125,
                           rot=dict(dims=32, base=10000.0)))


cfg = DictConfig(
    dict(
        vocab=32000, width=512, norm=dict(eps=1e-6), embedding=dict(scale=22.6), logit_softcap=50.0,
        layers=[_chunked(mlp=dict(kind="dense", ff=2048)), _windowed(mlp=_moe(512)), _chunked(kv_from=0, mlp=_moe(512)),
                _windowed(mlp=_moe(512))],
        initializer_range=0.02,
        # generation defaults
        is_encoder_decoder=False, max_length=256, do_sample=False, num_beams=1, temperature=1.0, top_k=50, top_p=1.0,
        use_cache=True, bos_token_id=1, eos_token_id=2, pad_token_id=0,
    )
)

model = LazyCall(NefelornForCausalLM)(cfg=cfg)
