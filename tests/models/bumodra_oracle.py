"""Plain, slow, float64 statement of the Bumodra mechanisms, one function per mechanism, token by token.

Written from the equations only; shares no code with ``libai_b200``.  Weights are a dict in checkpoint naming
(``l<i>.mix.q``, ``l<i>.mix.q.conv``, ``embed.norm`` …), the configuration is the ``config.json`` dictionary.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def short_conv_silu(xs, w):
    """xs [T, C] inputs over time, w [C, taps] (last column = current token); zeros before the start."""
    T, C = xs.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        acc = torch.zeros(C, dtype=F64)
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                acc = acc + w[:, j] * xs[src]
        out[t] = silu(acc)
    return out


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, D] (already unit / scaled), v [T, H, V], beta [T, H], g [T, H, D] → o [T, H, V]; state starts at 0."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].t() @ k[t, h])
            S[h] = S[h] + torch.outer(k[t, h], u)
            o[t, h] = S[h].t() @ q[t, h]
    return o


def delta_mixer(hs, w, p, m, eps, channel):
    """hs [T, width] → mixer output [T, width] for a ``delta`` (channel=False) or ``channel_delta`` mixer."""
    T = hs.shape[0]
    H, KH, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(hs @ w[p + "q"].t(), w[p + "q.conv"]).view(T, KH, D)
    k = short_conv_silu(hs @ w[p + "k"].t(), w[p + "k.conv"]).view(T, KH, D)
    v = short_conv_silu(hs @ w[p + "v"].t(), w[p + "v.conv"]).view(T, H, V)
    q = unit(q) * D ** -0.5
    k = unit(k)
    group = H // KH
    idx = torch.tensor([h // group for h in range(H)])
    q, k = q[:, idx], k[:, idx]
    beta = torch.sigmoid(hs @ w[p + "b"].t())
    rate = torch.exp(w[p + "A_log"])
    if channel:
        logits = (hs @ w[p + "a1"].t()) @ w[p + "a2"].t() + w[p + "dt_bias"]
        g = torch.exp(-rate[None, :, None] * softplus(logits.view(T, H, D)))
        gate = torch.sigmoid((hs @ w[p + "g1"].t()) @ w[p + "g2"].t())
    else:
        g = torch.exp(-rate * softplus(hs @ w[p + "a"].t() + w[p + "dt_bias"]))[:, :, None].expand(T, H, D)
        gate = silu(hs @ w[p + "g"].t())
    o = delta_rule(q, k, v, beta, g)
    o = rms_unit(o, eps) * w[p + "norm"] * gate.view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].t()


def latent_attention(hs, w, p, m, eps, window=None):
    T = hs.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    window = m["mask"]["size"] if window is None else window
    scale = m.get("scale", D ** -0.5)
    cq = plain_norm(hs @ w[p + "dq"].t(), w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].t()).view(T, H, D)
    c = plain_norm(hs @ w[p + "dkv"].t(), w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].t()).view(T, H, D)
    v = (c @ w[p + "uv"].t()).view(T, H, V)
    gate = torch.sigmoid(hs @ w[p + "g"].t())
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            pr = torch.softmax(s, 0)
            out[i, h] = (pr[:, None] * v[lo:i + 1, h]).sum(0) * gate[i, h]
    return out.reshape(T, H * V) @ w[p + "o"].t()


def feed_forward(hs, w, p):
    return (torch.relu(hs @ w[p + "up"].t()) ** 2) @ w[p + "down"].t()


def block_runs(cfg):
    """(block index, enters a pass) in execution order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def model_logits(cfg, weights, tokens, return_stream=False):
    """Whole sequence at once (every mechanism above is causal and starts from an empty state)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = zero_centred_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
    x0 = x.clone()
    stream = []
    for i, enters in block_runs(cfg):
        lc, p = cfg["layers"][i], f"l{i}."
        if enters:
            x = torch.cat([x, x0], -1) @ w["loop.in"].t()
        h = zero_centred_norm(x, w[p + "norm1"], eps)
        if lc["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", lc["mixer"], eps)
        else:
            y = delta_mixer(h, w, p + "mix.", lc["mixer"], eps, lc["type"] == "channel_delta")
        if lc.get("mlp"):
            y = y + feed_forward(h, w, p + "mlp.")
        x = x + y
        stream.append(x.clone())
    logits = zero_centred_norm(x, w["final.norm"], eps) @ w["head"].t()
    return (logits, torch.stack(stream)) if return_stream else logits


def greedy(cfg, weights, prompt, new_tokens):
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(model_logits(cfg, weights, seq)[-1].argmax()))
    return seq[len(prompt):]


# ------------------------------------------------------------------------------------------------ random models for the tests
def random_weights(cfg, seed=0, ranks=(6, 5)):
    gen = torch.Generator().manual_seed(seed)

    def mat(o, i, gain=1.0):
        return (torch.randn(o, i, generator=gen) * gain / math.sqrt(i)).to(torch.bfloat16).float()

    def vec(n, mean=0.0, std=0.3):
        return (mean + std * torch.randn(n, generator=gen)).to(torch.bfloat16).float()

    W, w = cfg["width"], {}
    w["embed"], w["embed.norm"] = mat(cfg["vocab"], W, math.sqrt(W)), vec(W)
    if cfg.get("loop"):
        w["loop.in"] = mat(W, 2 * W, 1.4)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", lc["mixer"]
        w[f"l{i}.norm1"] = vec(W)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if lc["type"] == "latent_attention":
            w[p + "dq"], w[p + "dq.norm"], w[p + "uq"] = mat(m["q_rank"], W), vec(m["q_rank"], 1.0), mat(H * D, m["q_rank"], 2.0)
            w[p + "dkv"], w[p + "dkv.norm"] = mat(m["kv_rank"], W), vec(m["kv_rank"], 1.0)
            w[p + "uk"], w[p + "uv"] = mat(H * D, m["kv_rank"], 2.0), mat(H * V, m["kv_rank"])
            w[p + "g"], w[p + "o"] = mat(H, W), mat(W, H * V)
        else:
            KH, taps = m["kv_heads"], m["conv"]
            for n, rows in (("q", KH * D), ("k", KH * D), ("v", H * V)):
                w[p + n], w[p + n + ".conv"] = mat(rows, W, 2.0), vec(rows * taps, 0.0, 0.5).view(rows, taps)
            w[p + "b"], w[p + "A_log"], w[p + "norm"] = mat(H, W, 2.0), vec(H, -1.0, 0.7), vec(V, 1.0)
            if lc["type"] == "channel_delta":
                w[p + "a1"], w[p + "a2"], w[p + "dt_bias"] = mat(ranks[0], W), mat(H * D, ranks[0], 2.0), vec(H * D, -1.0, 1.0)
                w[p + "g1"], w[p + "g2"] = mat(ranks[1], W), mat(H * V, ranks[1], 2.0)
            else:
                w[p + "a"], w[p + "dt_bias"], w[p + "g"] = mat(H, W, 2.0), vec(H, -1.0, 1.0), mat(H * V, W, 2.0)
            w[p + "o"] = mat(W, H * V)
        if lc.get("mlp"):
            w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"] = mat(lc["mlp"]["ff"], W, 1.4), mat(W, lc["mlp"]["ff"])
    w["final.norm"], w["head"] = vec(W), mat(cfg["vocab"], W)
    return w


def attention_cfg(heads=3, dim=8, vdim=12, q_rank=10, kv_rank=9, window=5, scale=None, ff=24):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window}}
    if scale is not None:
        m["scale"] = scale
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_cfg(channel=False, heads=4, kv_heads=2, dim=8, vdim=12, conv=3, ff=24):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    return {"type": "channel_delta" if channel else "delta", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_cfg(layers, width=24, vocab=50, loop=None, eps=1e-5):
    cfg = {"architecture": "Bumodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = loop
    return cfg
