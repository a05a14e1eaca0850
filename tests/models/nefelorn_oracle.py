"""A plain, slow restatement of the Nefelorn design in float64, token by token, one function per mechanism.  It shares no code
with the package: the tests compare the framework's operators, layers, cache and scheduler against it.

Notation.  ``x`` is the residual stream of one sequence ``[n, width]``; positions count from 0.  Linear maps are stored
``[out, in]`` and applied as ``W @ v``.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------------------ small pieces
def dyt(v, w, b, alpha):
    """Dynamic Tanh: an elementwise squashing with a learned slope, then scale and shift."""
    return torch.tanh(alpha * v) * w + b


def rms_divide(v, eps):
    return v / torch.sqrt((v * v).mean() + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def rotary_table(rot):
    """Angular frequency of every rotated pair and the common factor on cos / sin."""
    dims, base = rot["dims"], float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    factor_cs = 1.0
    sc = rot.get("scaling")
    if sc:
        def dim_of(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
        out = []
        for i, f in enumerate(freqs):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
        freqs = out
        factor_cs = 0.1 * math.log(sc["factor"]) + 1.0
    return freqs, factor_cs


def rotate_head(vec, position, rot):
    """One head ``[dim]``: channel i is paired with channel i + dims/2 for i < dims/2; the other channels pass."""
    dims = rot["dims"]
    freqs, fcs = rotary_table(rot)
    out = vec.clone()
    for i in range(dims // 2):
        a = position * freqs[i]
        c, s = math.cos(a) * fcs, math.sin(a) * fcs
        u, v = vec[i], vec[i + dims // 2]
        out[i] = u * c - v * s
        out[i + dims // 2] = v * c + u * s
    return out


def sees_chunk(i, j, size):
    return j <= i and i // size == j // size


def sees_window(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def softmax_read(q_head, keys, values, scale):
    """One query head over the keys / values it sees (lists of vectors)."""
    scores = torch.stack([(q_head * k).sum() * scale for k in keys])
    p = torch.exp(scores - scores.max())
    p = p / p.sum()
    return sum(pj * v for pj, v in zip(p, values))


# ------------------------------------------------------------------------------------------------------------------ mixers
def attention_keys(h, W, p, m, eps, kind):
    """Keys (as the cache holds them) and values of one block for the normed inputs ``h`` ``[n, width]``:
    lists over positions of ``[G, dim]`` / ``[G, vdim]``."""
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    ks, vs = [], []
    for t in range(h.shape[0]):
        k = W[p + "mix.k"] @ h[t]
        v = (W[p + "mix.v"] @ h[t]).view(G, V)
        if kind == "attention":
            k = rms_divide(k, eps) * W[p + "mix.k.norm"]
            k = torch.stack([rotate_head(k.view(G, D)[g], t, m["rot"]) for g in range(G)])
        else:
            k = torch.stack([rms_divide(rotate_head(k.view(G, D)[g], t, m["rot"]), eps) for g in range(G)])
        ks.append(k)
        vs.append(v)
    return ks, vs


def attention_block(h, W, p, m, eps, kind, ks, vs):
    """Output of the mixer (before its closing norm) for every position; ``ks`` / ``vs`` are this block's own keys or the ones
    of the block it reads."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    out = torch.zeros(n, W[p + "mix.o"].shape[0], dtype=F64)
    for t in range(n):
        q = W[p + "mix.q"] @ h[t]
        if kind == "attention":
            q = rms_divide(q, eps) * W[p + "mix.q.norm"]
            q = torch.stack([rotate_head(q.view(H, D)[hh], t, m["rot"]) for hh in range(H)])
            seen = [j for j in range(t + 1) if sees_chunk(t, j, m["mask"]["size"])]
        else:
            q = torch.stack([rms_divide(rotate_head(q.view(H, D)[hh], t, m["rot"]), eps) for hh in range(H)])
            seen = [j for j in range(t + 1) if sees_window(t, j, m["mask"]["size"], m["mask"].get("keep_first", 0))]
        heads = []
        for hh in range(H):
            g = hh // (H // G)
            heads.append(softmax_read(q[hh], [ks[j][g] for j in seen], [vs[j][g] for j in seen], m["scale"]))
        heads = torch.stack(heads)                              # [H, V]
        if kind == "attention":
            heads = heads * torch.sigmoid(W[p + "mix.g"] @ h[t])[:, None]
        out[t] = W[p + "mix.o"] @ heads.reshape(-1)
    return out


# ----------------------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(v, W, p):
    return W[p + "mlp.down"] @ gelu_erf(W[p + "mlp.up"] @ v)


def router_choice(v, W, p, r):
    """Chosen experts (largest scores first) and their weights."""
    s = torch.sigmoid(W[p + "mlp.router"] @ v)
    order = sorted(range(r["experts"]), key=lambda e: (-float(s[e]), e))[: r["top"]]
    total = sum(s[e] for e in order) + 1e-20
    return order, [s[e] / total * r["scale"] for e in order]


def moe_ff(v, W, p, r):
    chosen, weights = router_choice(v, W, p, r)
    out = 0
    for e, w in zip(chosen, weights):
        q = p + f"mlp.e{e}."
        out = out + w * (W[q + "down"] @ (silu(W[q + "gate"] @ v) * (W[q + "up"] @ v)))
    return out


# ------------------------------------------------------------------------------------------------------------- whole model
def forward(cfg, weights, tokens, window_shift=0, chunk_shift=0, keep_shift=0):
    """Logits ``[n, vocab]`` and the stream after every block, for one sequence fed whole.  The ``*_shift`` arguments move the
    masks' constants by that much — a deliberately wrong oracle that a test compares against to show that it would notice."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][tokens] * cfg["embedding"]["scale"]
    n = x.shape[0]
    streams, cache = [], {}
    for li, lc in enumerate(cfg["layers"]):
        p = f"l{li}."
        m = dict(lc["mixer"])
        m["mask"] = dict(m["mask"])
        if lc["type"] == "attention":
            m["mask"]["size"] += chunk_shift
        else:
            m["mask"]["size"] += window_shift
            m["mask"]["keep_first"] = m["mask"].get("keep_first", 0) + keep_shift
        nrm = lambda name, v: dyt(v, W[p + name], W[p + name + ".b"], W[p + name + ".alpha"])
        h = torch.stack([nrm("norm1", x[t]) for t in range(n)])
        if "kv_from" in m:
            ks, vs = cache[m["kv_from"]]
        else:
            ks, vs = attention_keys(h, W, p, m, eps, lc["type"])
            cache[li] = (ks, vs)
        y = attention_block(h, W, p, m, eps, lc["type"], ks, vs)
        x = x + torch.stack([nrm("norm1b", y[t]) for t in range(n)])
        ml = lc.get("mlp")
        if ml:
            rows = []
            for t in range(n):
                v = nrm("norm2", x[t])
                rows.append(nrm("norm2b", dense_ff(v, W, p) if ml["kind"] == "dense" else moe_ff(v, W, p, ml["router"])))
            x = x + torch.stack(rows)
        streams.append(x.clone())
    hfin = dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    logits = hfin @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, streams


def greedy(cfg, weights, prompt, new_tokens):
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, weights, seq)[0][-1].argmax()))
    return seq[len(prompt):]


# ------------------------------------------------------------------------------------------------------- configurations
def rot_cfg(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def chunk_attention_cfg(heads=4, kv_heads=2, dim=8, vdim=8, chunk=5, rot=None, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
         "rot": rot or rot_cfg(dim, 100.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}),
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def window_attention_cfg(heads=4, kv_heads=1, dim=8, vdim=4, window=6, keep_first=2, rot=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "keep_first": keep_first},
         "rot": rot or rot_cfg(dim // 2, 1000.0), "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def dense_cfg(ff=24):
    return {"kind": "dense", "ff": ff}


def moe_cfg(ff=8, experts=6, top=2, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def model_cfg(layers, vocab=50, width=16, embedding_scale=3.0, softcap=20.0, eps=1e-5):
    return {"architecture": "Nefelorn", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale},
            "norm": {"eps": eps}, "logit_softcap": softcap, "layers": layers}


def random_weights(cfg, seed=0, spread=1.0):
    """Checkpoint tensors (names as in a checkpoint folder) with values that survive a round trip through bfloat16."""
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s * spread / math.sqrt(i)).to(torch.bfloat16).to(F64)

    def vecn(n, centre, s):
        return (centre + s * torch.randn(n, generator=g)).to(torch.bfloat16).to(F64)

    W = {"embed": mat(cfg["vocab"], width, math.sqrt(width) / 3.0), "head": mat(cfg["vocab"], width, 2.0)}

    def norm(name):
        W[name] = vecn(width, 1.0, 0.2)
        W[name + ".b"] = vecn(width, 0.0, 0.1)
        W[name + ".alpha"] = (0.4 + 0.4 * torch.rand((), generator=g)).to(torch.bfloat16).to(F64)

    norm("final.norm")
    for li, lc in enumerate(cfg["layers"]):
        p, m = f"l{li}.", lc["mixer"]
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        norm(p + "norm1")
        norm(p + "norm1b")
        W[p + "mix.q"] = mat(H * D, width, 2.0)
        W[p + "mix.o"] = mat(width, H * V, 2.0)
        if "kv_from" not in m:
            W[p + "mix.k"] = mat(G * D, width, 2.0)
            W[p + "mix.v"] = mat(G * V, width, 2.0)
        if lc["type"] == "attention":
            W[p + "mix.q.norm"] = vecn(H * D, 1.0, 0.3)
            if "kv_from" not in m:
                W[p + "mix.k.norm"] = vecn(G * D, 1.0, 0.3)
            W[p + "mix.g"] = mat(H, width, 2.0)
        ml = lc.get("mlp")
        if ml:
            norm(p + "norm2")
            norm(p + "norm2b")
            if ml["kind"] == "dense":
                W[p + "mlp.up"] = mat(ml["ff"], width, 2.0)
                W[p + "mlp.down"] = mat(width, ml["ff"], 2.0)
            else:
                W[p + "mlp.router"] = mat(ml["router"]["experts"], width, 3.0)
                for e in range(ml["router"]["experts"]):
                    W[p + f"mlp.e{e}.gate"] = mat(ml["expert"]["ff"], width, 2.0)
                    W[p + f"mlp.e{e}.up"] = mat(ml["expert"]["ff"], width, 2.0)
                    W[p + f"mlp.e{e}.down"] = mat(width, ml["expert"]["ff"], 2.0)
    return W
