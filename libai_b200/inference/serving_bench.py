"""Prefill / decode throughput of the stateful sequence-mixer model (Bumodra) beside Llama at equal width, depth and
feed-forward size, random weights, one GPU.  ``bench.py --serving`` prints the result as one JSON line; ``--serving-kernels``
adds device times of the individual kernels of one block at the same sizes with their roofline fractions.

Timing: CUDA events on the launching stream after warm-up steps, a synchronize on both sides, an L2 flush (a write larger
than L2) between timed iterations of the kernel table.
"""
from __future__ import annotations

import json
import os
import time

import torch

SIZES = {
    # name: width, ff, heads, head dim, latent ranks, window, blocks
    "w1024": dict(width=1024, ff=4096, heads=8, dim=128, q_rank=512, kv_rank=256, window=512, blocks=4, vocab=32000),
    "w2048": dict(width=2048, ff=8192, heads=16, dim=128, q_rank=768, kv_rank=512, window=1024, blocks=4, vocab=32000),
}


def bumodra_config(s):
    att = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": s["ff"]},
           "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "q_rank": s["q_rank"], "kv_rank": s["kv_rank"],
                     "mask": {"size": s["window"]}, "scale": s["dim"] ** -0.5}}
    delta = {"type": "delta", "mlp": {"kind": "dense", "ff": s["ff"]},
             "mixer": {"heads": s["heads"], "kv_heads": s["heads"] // 2, "dim": s["dim"], "vdim": s["dim"], "conv": 4}}
    chan = {"type": "channel_delta", "mlp": {"kind": "dense", "ff": s["ff"]},
            "mixer": {"heads": s["heads"], "kv_heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "conv": 4,
                      "decay_rank": 64, "gate_rank": 64}}
    kinds = [att, delta, delta, chan]
    return dict(vocab=s["vocab"], width=s["width"], norm={"eps": 1e-6}, layers=[kinds[i % 4] for i in range(s["blocks"])])


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]) * 1e9, float(p["bf16_tflops"]) * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


def _time(fn, warmup=3, iters=10, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def build_models(s, device="cuda"):
    from libai_b200.config import DictConfig
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import BumodraForCausalLM, LlamaForCausalLM

    with param_defaults(dtype=torch.bfloat16, device=device, seed=1):
        bum = BumodraForCausalLM(DictConfig(bumodra_config(s))).eval()
        # SwiGLU has three matrices where the dense feed-forward has two: 2/3 of ff gives the same parameter count
        llama = LlamaForCausalLM(DictConfig(dict(
            hidden_layers=s["blocks"], vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=(2 * s["ff"] // 3 + 127) // 128 * 128,
            num_attention_heads=s["heads"] if s["width"] // s["heads"] in (64, 128) else s["width"] // 128,
            max_position_embeddings=8192, rms_norm_eps=1e-6, initializer_range=0.02, use_scaled_init_for_output_weights=True,
            scale_mask_softmax_fusion=False, amp_enabled=False))).eval()
    return bum.cuda(), llama.cuda()            # .cuda(): the rotary tables are buffers built on the host


@torch.no_grad()
def throughput(s, batch, prompt, new_tokens, steps, warmup):
    from libai_b200.inference.scheduler import RequestScheduler

    bum, llama = build_models(s)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(1, s["vocab"], (batch, prompt), generator=gen)
    out = {}
    # ---- the stateful model through its scheduler: one ragged prefill step, then single-token steps
    sched = RequestScheduler(bum)
    prompts = [row.tolist() for row in ids]

    def prefill():
        sched.step([(("p", i), p, [len(p) - 1]) for i, p in enumerate(prompts)])
        sched.finish([("p", i) for i in range(batch)])

    out["bumodra_prefill_ms"] = _time(prefill, warmup, steps)
    sched.step([(("d", i), p, []) for i, p in enumerate(prompts)])
    entries = [(("d", i), [7], [0]) for i in range(batch)]
    out["bumodra_decode_ms"] = _time(lambda: sched.step(entries), warmup, new_tokens)
    sched.finish([("d", i) for i in range(batch)])
    # ---- Llama: the prompt through the packed flash-attention path (no cache), single tokens against a key/value cache of
    # `prompt` positions per layer (filled with random values: only the time matters) as Generator.generate drives them
    dev_ids = ids.cuda()
    out["llama_prefill_ms"] = _time(lambda: llama(dev_ids), warmup, steps)
    a, d = llama.model.layers[0].self_attn.local_heads, llama.model.layers[0].self_attn.head_size
    one = dev_ids[:, :1].contiguous()

    def llama_decode():
        llama(one, use_cache=True)

    def fill_cache():
        llama.set_cache([(torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16),
                          torch.randn(batch, a, prompt, d, device="cuda").to(torch.bfloat16)) for _ in range(s["blocks"])])

    fill_cache()
    out["llama_decode_ms"] = _time(llama_decode, warmup, new_tokens)
    llama.set_cache(None)
    for name in ("bumodra", "llama"):
        out[f"{name}_prefill_tokens_per_s"] = batch * prompt / out[f"{name}_prefill_ms"] * 1e3
        out[f"{name}_decode_tokens_per_s"] = batch / out[f"{name}_decode_ms"] * 1e3
    out["params_bumodra"] = sum(p.numel() for p in bum.parameters())
    out["params_llama"] = sum(p.numel() for p in llama.parameters())
    return out


@torch.no_grad()
def kernel_table(s, batch, prompt):
    """Device time of every kernel of the mixers at these sizes (prefill rows = batch·prompt; decode rows = batch), with the
    bytes / FLOPs the operation needs and the fraction of the measured roofline that this is."""
    from libai_b200.inference.ragged import RaggedBatch
    from libai_b200.ops import functional as OF
    from libai_b200.ops import seq_functional as SF

    hbm, flops, src = _peaks()
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, D, W, C = s["heads"], s["dim"], s["window"], s["kv_rank"]
    rows = []

    def add(name, ms, bytes_=0.0, fl=0.0):
        ideal = max(bytes_ / hbm, fl / flops) * 1e3
        rows.append(dict(kernel=name, ms=round(ms, 4), ideal_ms=round(ideal, 5), roofline_fraction=round(ideal / ms, 4),
                         bound="memory" if bytes_ / hbm >= fl / flops else "tensor"))

    for phase, lens, past in (("prefill", [prompt] * batch, [0] * batch), ("decode", [1] * batch, [prompt] * batch)):
        rb = RaggedBatch(lens, list(range(batch)), past, dev)
        T = rb.tokens
        x = torch.randn(T, s["width"], device=dev)
        w = torch.zeros(s["width"], dtype=bf, device=dev)
        h = torch.empty(T, s["width"], dtype=bf, device=dev)
        add(f"{phase}: rms norm fp32→bf16", _time(lambda: SF.rms_norm_rows(x, w, offset=1.0, eps=1e-6, out=h), flush=flush), T * s["width"] * 6)
        # delta rule: convolution, scan, gated norm
        KH = H // 2
        Cq = 2 * KH * D + H * D
        qkv = torch.randn(T, Cq, device=dev).to(bf)
        cw = torch.randn(Cq, 4, device=dev).to(bf)
        tail = torch.zeros(batch, 3, Cq, dtype=bf, device=dev)
        conv = torch.empty_like(qkv)
        add(f"{phase}: short conv + silu", _time(lambda: SF.short_conv(qkv, cw, tail, rb, conv), flush=flush), T * Cq * 4)
        a, b = torch.randn(T, H, device=dev).to(bf), torch.randn(T, H, device=dev).to(bf)
        A_log, dtb = torch.zeros(H, dtype=bf, device=dev), torch.zeros(H, dtype=bf, device=dev)
        S = torch.zeros(batch, H, D, D, device=dev)
        state_bytes = batch * H * D * D * 4 * (2 if phase == "decode" else 1)
        add(f"{phase}: delta scan (per-head decay)", _time(lambda: SF.delta_scan(conv, KH * D, 2 * KH * D, a, b, A_log, dtb, S, rb, KH, False), flush=flush),
            T * (Cq * 2 + H * D * 4) + state_bytes, 0.0)
        o = torch.randn(T, H * D, device=dev)
        g, nw, y = torch.randn(T, H * D, device=dev).to(bf), torch.ones(D, dtype=bf, device=dev), torch.empty(T, H * D, dtype=bf, device=dev)
        add(f"{phase}: gated rms norm", _time(lambda: SF.gated_rmsnorm(o, g, nw, 1e-6, 0, y, H, D), flush=flush), T * H * D * 8)
        # latent attention
        ring = torch.randn(batch, W, C, device=dev).to(bf)
        c = torch.randn(T, C, device=dev).to(bf)
        q = torch.randn(T, H * D, device=dev).to(bf)
        gate = torch.randn(T, H, device=dev).to(bf)
        if phase == "prefill":
            kv = torch.randn(rb.ext(W).rows, 2 * H * D, device=dev).to(bf)
            pairs = sum(min(t + 1, W) for t in range(prompt)) * batch
            add("prefill: window attention", _time(lambda: SF.window_attention(q, kv, gate, rb, y, H, D, D, W, D ** -0.5), flush=flush),
                T * H * D * 4 + kv.numel() * 2, pairs * H * D * 4.0)
            qkv4 = torch.randn(batch, prompt, H, 3 * D, device=dev).to(bf)
            add("prefill: Llama causal flash attention (same heads, full context)",
                _time(lambda: OF.attention_qkvpacked(qkv4, causal=True, scale=D ** -0.5), flush=flush),
                qkv4.numel() * 2 + T * H * D * 2, batch * prompt * (prompt + 1) / 2 * H * D * 4.0)
        else:
            qa = torch.randn(batch, H, C, device=dev)
            add("decode: absorbed latent attention", _time(lambda: SF.latent_decode(qa, ring, c, rb, W, D ** -0.5), flush=flush),
                batch * W * C * 2 + batch * H * C * 8)
            k = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            v = torch.randn(batch, H, prompt, D, device=dev).to(bf)
            q1 = torch.randn(batch, H, 1, D, device=dev).to(bf)
            add("decode: Llama attention over its key/value cache",
                _time(lambda: OF.attention(q1, k, v, causal=False, scale=D ** -0.5), flush=flush), k.numel() * 4)
    return {"peaks": src, "hbm_bytes_per_s": hbm, "bf16_flops": flops, "rows": rows}


def main(args):
    assert torch.cuda.is_available(), "the serving bench needs a GPU"
    from libai_b200 import ops

    ops.reset_launch_count()
    result = {"metric": "prefill / decode tokens per second, Bumodra beside Llama at equal width, depth and parameter count",
              "dtype": "bf16", "data": "synthetic tokens, random-init weights", "n_gpus": 1, "sizes": {}}
    for name in (args.serving_sizes.split(",") if args.serving_sizes else list(SIZES)):
        s = SIZES[name]
        r = throughput(s, args.serving_batch, args.serving_prompt, new_tokens=max(args.steps, 8), steps=max(args.steps // 2, 3),
                       warmup=max(args.warmup, 3))
        if args.serving_kernels:
            r["kernels"] = kernel_table(s, args.serving_batch, args.serving_prompt)
        result["sizes"][name] = {"config": {k: v for k, v in s.items()}, "batch": args.serving_batch, "prompt": args.serving_prompt, **r}
        torch.cuda.empty_cache()
    result["gpu_launches"] = ops.launch_count()
    print(json.dumps(result))
