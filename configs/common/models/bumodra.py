"""A small Bumodra causal LM: latent sliding-window attention, two gated delta-rule blocks and a per-channel-decay one, the first
two blocks looped twice.  Checkpoint folders carry their own ``config.json``; this record is for random-init runs."""
from libai_b200.config import DictConfig, LazyCall
from libai_b200.models import BumodraForCausalLM


def _ff(n):
    return dict(kind="dense", ff=n)


cfg = DictConfig(
    dict(
        vocab=32000, width=512, norm=dict(eps=1e-6),
        layers=[
            dict(type="latent_attention", mlp=_ff(2048),
                 mixer=dict(heads=8, dim=64, vdim=64, q_rank=256, kv_rank=128, mask=dict(size=256), scale=0.125)),
            dict(type="delta", mlp=_ff(2048), mixer=dict(heads=8, kv_heads=4, dim=64, vdim=64, conv=4)),
            dict(type="delta", mlp=_ff(2048), mixer=dict(heads=8, kv_heads=4, dim=64, vdim=64, conv=4)),
            dict(type="channel_delta", mlp=_ff(2048),
                 mixer=dict(heads=8, kv_heads=8, dim=64, vdim=64, conv=4, decay_rank=32, gate_rank=32)),
        ],
        loop=dict(start=0, stop=2, times=2),
        initializer_range=0.02,
        # generation defaults
        is_encoder_decoder=False, max_length=256, do_sample=False, num_beams=1, temperature=1.0, top_k=50, top_p=1.0,
        use_cache=True, bos_token_id=1, eos_token_id=2, pad_token_id=0,
    )
)

model = LazyCall(BumodraForCausalLM)(cfg=cfg)
