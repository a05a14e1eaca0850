"""Nefelorn against a plain float64 oracle (``nefelorn_oracle.py``): every mechanism alone, whole prompts, decoding through the
key/value rings, prompt portions, ragged batches, slot reuse, mask edges with a sharp softmax, long decoding over many ring
wraps, odd sizes, generation.

The CPU parametrisation exercises the framework's PyTorch operators; the ``cuda`` one (marked ``gpu``) the sm_100a kernels.
"""
import importlib.util
import json
import math
import os

import pytest
import torch

from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.scheduler import RequestScheduler
from libai_b200.layers import DynamicTanh, MoEFeedForward
from libai_b200.layers._param import param_defaults
from libai_b200.models.utils.model_loader.auto import load_pretrained
from libai_b200.ops import kv_functional as KF

from . import nefelorn_oracle as O

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]
REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel_err(got, want):
    """Error of logits the way a user sees it: mean removed, RMS over the vocabulary, relative to the RMS of the target."""
    got, want = got.detach().cpu().double(), want.double()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    scale = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return float(d.pow(2).mean(-1).sqrt().max() / scale)


def save_model(tmp_path, cfg, weights, name="m"):
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def make(tmp_path, cfg, device, dtype=torch.float32, seed=0, weights=None):
    weights = weights if weights is not None else O.random_weights(cfg, seed)
    return load_pretrained(save_model(tmp_path, cfg, weights), dtype=dtype, device=device), weights


def run_schedule(model, prompts, cuts, **kw):
    """Feed ``prompts`` together: step s brings ``cuts[i][s]`` tokens of prompt i (requests that have nothing left drop out).
    Returns per prompt the logits of all its positions."""
    sched = RequestScheduler(model, **kw)
    at = [0] * len(prompts)
    got = [[] for _ in prompts]
    for s in range(max(len(c) for c in cuts)):
        entries, who = [], []
        for i, p in enumerate(prompts):
            if s < len(cuts[i]):
                n = cuts[i][s]
                entries.append((("r", i), p[at[i]:at[i] + n], list(range(n))))
                who.append((i, n))
                at[i] += n
        logits = sched.step(entries)
        o = 0
        for i, n in who:
            got[i].append(logits[o:o + n].clone())
            o += n
        sched.finish([("r", i) for i, p in enumerate(prompts) if at[i] == len(p)])
    assert sched.cache.live() == 0
    return [torch.cat(g) for g in got]


def tokens(n, vocab=50, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def mixed_cfg(**kw):
    """Every branch once: a chunked block with a dense feed-forward, a kept-first window block with experts, a block that
    reads the first block's keys under a chunk of another size and has no feed-forward, a window block that keeps nothing."""
    layers = [O.chunk_attention_cfg(heads=4, kv_heads=2, dim=8, vdim=6, chunk=5, mlp=O.dense_cfg(20)),
              O.window_attention_cfg(heads=4, kv_heads=1, dim=8, vdim=4, window=6, keep_first=2, mlp=O.moe_cfg()),
              O.chunk_attention_cfg(heads=4, kv_heads=2, dim=8, vdim=6, chunk=7, kv_from=0, mlp=None),
              O.window_attention_cfg(heads=3, kv_heads=3, dim=4, vdim=8, window=3, keep_first=0, rot=O.rot_cfg(4, 50.0),
                                     mlp=O.moe_cfg(ff=4, experts=3, top=1, scale=1.0))]
    return O.model_cfg(layers, **kw)


# ------------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("device", DEVICES)
def test_dynamic_tanh_around_the_residual(device):
    g = torch.Generator().manual_seed(1)
    n = 20
    x, y = torch.randn(5, n, generator=g), 3.0 * torch.randn(5, n, generator=g)
    with param_defaults(dtype=torch.float32, device=device):
        post, nxt = DynamicTanh(n), DynamicTanh(n)
    with torch.no_grad():
        for mod, a in ((post, 0.3), (nxt, 1.7)):
            mod.weight.copy_(torch.randn(n, generator=g))
            mod.bias.copy_(torch.randn(n, generator=g))
            mod.alpha.fill_(a)
    xs, h = x.clone().to(device), torch.empty(5, n, device=device)
    KF.dyt_residual(xs, y.to(device), post=post.triple(), nxt=nxt.triple(), h=h)
    P = [t.detach().cpu().double() for t in post.triple()]
    N = [t.detach().cpu().double() for t in nxt.triple()]
    want_x = x.double() + O.dyt(y.double(), *P)
    assert torch.allclose(xs.cpu().double(), want_x, atol=1e-5)
    assert torch.allclose(h.cpu().double(), O.dyt(want_x, *N), atol=1e-5)
    # a norm that divided by a root mean square would be far away
    assert not torch.allclose(h.cpu().double(), want_x / want_x.pow(2).mean(-1, keepdim=True).sqrt() * N[0] + N[1], atol=1e-2)
    out = torch.empty(5, n, device=device)
    nxt.rows(xs, out)
    assert torch.allclose(out, h)


@pytest.mark.parametrize("rot", [O.rot_cfg(8, 100.0), O.rot_cfg(16, 250.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}),
                                 O.rot_cfg(32, 1e4, {"factor": 16.0, "original": 64, "fast": 2.0, "slow": 0.5}),
                                 O.rot_cfg(8, 10.0, {"factor": 2.0, "original": 10, "fast": 1.0, "slow": 0.1}),
                                 O.rot_cfg(8, 10.0, {"factor": 2.0, "original": 1000, "fast": 1.0, "slow": 1e-3})])
def test_rotary_frequencies(rot):
    freq, ms = KF.rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    want, want_ms = O.rotary_table(rot)
    assert torch.allclose(freq.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
    assert abs(ms - want_ms) < 1e-12
    if rot.get("scaling") and rot["scaling"]["original"] < 1000:        # the last case clamps every dimension to "unchanged"
        plain, _ = O.rotary_table({"dims": rot["dims"], "base": rot["base"]})
        assert not torch.allclose(freq.double(), torch.tensor(plain, dtype=torch.float64), rtol=1e-3)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("mode", ["full", "head_unit"])
@pytest.mark.parametrize("dims,D", [(8, 8), (4, 12), (0, 6)])
def test_query_key_preparation(device, mode, dims, D):
    g = torch.Generator().manual_seed(dims + D)
    H, G, eps = 3, 1, 1e-3
    lens, past = [4, 1, 3], [0, 37, 5]
    T = sum(lens)
    q, k = torch.randn(T, H * D, generator=g), torch.randn(T, G * D, generator=g)
    qw, kw = torch.randn(H * D, generator=g), torch.randn(G * D, generator=g)
    rot = O.rot_cfg(dims, 30.0, {"factor": 3.0, "original": 8, "fast": 3.0, "slow": 1.0}) if dims else {"dims": 0, "base": 1.0}
    freq, ms = KF.rotary_frequencies(dims, rot["base"], rot.get("scaling")) if dims else (torch.zeros(0), 1.0)
    rb = RaggedBatch(lens, [0, 1, 2], past, device)
    qd, kd = q.clone().to(device), k.clone().to(device)
    KF.qk_prepare(qd, kd, qw.to(device), kw.to(device), freq.to(device), ms, rb, H, G, D, eps, mode == "full", mode == "head_unit")
    pos = [p + t for n, p in zip(lens, past) for t in range(n)]
    for r in range(T):
        for src, got, w, heads in ((q, qd, qw, H), (k, kd, kw, G)):
            v = src[r].double()
            if mode == "full":
                v = O.rms_divide(v, eps) * w.double()
            rows = []
            for hh in range(heads):
                u = v.view(heads, D)[hh]
                u = O.rotate_head(u, pos[r], rot) if dims else u
                rows.append(O.rms_divide(u, eps) if mode == "head_unit" else u)
            assert torch.allclose(got[r].cpu().double(), torch.cat(rows), atol=2e-5), (r, mode)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,top", [(6, 2), (5, 1), (4, 4), (40, 3)])
@torch.no_grad()
def test_router_and_both_expert_forms(device, experts, top):
    g = torch.Generator().manual_seed(experts)
    width, ff, T, scale = 16, 8, 23, 1.7
    cfg = O.model_cfg([O.chunk_attention_cfg(mlp=O.moe_cfg(ff, experts, top, scale))], width=width)
    W = O.random_weights(cfg, seed=experts)
    with param_defaults(dtype=torch.float32, device=device):
        moe = MoEFeedForward(width, ff, experts, top, router_scale=scale)
    with torch.no_grad():
        moe.router.copy_(W["l0.mlp.router"])
        moe.gate_up.copy_(torch.stack([torch.cat([W[f"l0.mlp.e{e}.gate"], W[f"l0.mlp.e{e}.up"]]) for e in range(experts)]))
        moe.down.copy_(torch.stack([W[f"l0.mlp.e{e}.down"] for e in range(experts)]))
    h = torch.randn(T, width, generator=g)
    want = torch.stack([O.moe_ff(h[t].double(), W, "l0.", cfg["layers"][0]["mlp"]["router"]) for t in range(T)])
    idx, wts = KF.moe_route(h.to(device), moe.router, top, scale)
    for t in range(T):
        chosen, weights = O.router_choice(h[t].double(), W, "l0.", cfg["layers"][0]["mlp"]["router"])
        assert idx[t].tolist() == chosen
        assert torch.allclose(wts[t].cpu().double(), torch.stack(weights), atol=1e-6)
        assert abs(float(wts[t].sum()) - scale) < 1e-5
    y, pos, cw = moe(h.to(device), graph_safe=True)
    assert pos is None and torch.allclose(y.cpu().double(), want, atol=1e-4)
    ys, pos, cw = moe(h.to(device))
    assert pos is not None and sorted(pos.reshape(-1).tolist()) == list(range(T * top))
    x = torch.zeros(T, width, device=device)
    with param_defaults(dtype=torch.float32, device=device):
        ident = DynamicTanh(width)
    with torch.no_grad():
        ident.alpha.fill_(1e-3)                                 # tanh(a v) / a ≈ v
        ident.weight.fill_(1e3)
    KF.dyt_residual(x, ys, post=ident.triple(), pos=pos, cw=cw)
    assert torch.allclose(x.cpu().double(), want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("device", DEVICES)
def test_activations_and_softcap(device):
    v = torch.linspace(-6, 6, 101)[None, :].to(device)
    out = torch.empty_like(v)
    KF.act_rows(v, out, KF.ACT_GELU)
    assert torch.allclose(out.cpu().double(), O.gelu_erf(v.cpu().double()), atol=1e-6)
    tanh_form = 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    assert float((out - tanh_form).abs().max()) > 1e-4          # the erf form, not its tanh approximation
    both = torch.cat([v, 2 * v], 1).contiguous()
    KF.act_rows(both, out, KF.ACT_SILU, gated=True)
    assert torch.allclose(out.cpu().double(), O.silu(v.cpu().double()) * 2 * v.cpu().double(), atol=1e-5)
    l = (10 * v).float().contiguous()
    KF.softcap(l, 7.0)
    assert torch.allclose(l.cpu().double(), 7.0 * torch.tanh(10 * v.cpu().double() / 7.0), atol=1e-5)


# ------------------------------------------------------------------------------------------------- whole prompts, decoding
@pytest.mark.parametrize("device", DEVICES)
def test_whole_prompt_with_streams(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(19)
    want, streams = O.forward(cfg, W, toks)
    taps = []
    cache = model.state_cache()
    slots = cache.allocate(1)
    got = model.step(torch.tensor(toks, device=device), RaggedBatch([len(toks)], slots, [0], device),
                     tap=lambda i, x: taps.append(x.detach().cpu().double().clone()))
    cache.free(slots)
    for i, (a, b) in enumerate(zip(taps, streams)):
        assert torch.allclose(a, b, atol=2e-4), f"stream after block {i}"
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_prefill_against_token_by_token(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(26, seed=3)
    want, _ = O.forward(cfg, W, toks)
    whole, = run_schedule(model, [toks], [[len(toks)]])
    single, = run_schedule(model, [toks], [[1] * len(toks)])
    mixed, = run_schedule(model, [toks], [[9] + [1] * 17])
    for got in (whole, single, mixed):
        assert rel_err(got, want) < 1e-4
    assert rel_err(single, whole.cpu()) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cuts", [[2] * 15, [3, 7, 2, 11, 7], [13, 2, 2, 13], [1, 29], [29, 1]])
def test_prompt_portions(device, tmp_path, cuts):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(30, seed=5)
    want, _ = O.forward(cfg, W, toks)
    got, = run_schedule(model, [toks], [cuts])
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_ragged_batches_against_each_alone(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    prompts = [tokens(n, seed=n) for n in (1, 17, 4, 30, 9)]
    want = [O.forward(cfg, W, p)[0] for p in prompts]
    cuts = [[1], [12] + [1] * 5, [2, 1, 1], [21] + [1] * 9, [9]]
    together = run_schedule(model, prompts, cuts)
    for i, p in enumerate(prompts):
        alone, = run_schedule(model, [p], [cuts[i]])
        assert rel_err(together[i], want[i]) < 1e-4
        assert rel_err(together[i], alone.cpu()) < 1e-5
    # unequal portions in one step: long and short prompt pieces beside single tokens
    cuts2 = [[1], [5, 12], [1, 3], [2, 20, 8], [4, 1, 4]]
    for got, w in zip(run_schedule(model, prompts, cuts2), want):
        assert rel_err(got, w) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_slots_are_reused_without_clearing(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    sched = RequestScheduler(model)
    a, b, c = tokens(23, seed=1), tokens(8, seed=2), tokens(15, seed=3)
    sched.step([("a", a, []), ("b", b, [])])
    slot_a = sched.slot_of["a"]
    sched.finish(["a"])
    got = sched.step([("c", c[:6], list(range(6)))])               # takes a's slot, whose rings are full of a's rows
    assert sched.slot_of["c"] == slot_a
    got = torch.cat([got] + [sched.step([("c", [t], [0]), ("b", [1], [])]) for t in c[6:]])
    assert rel_err(got, O.forward(cfg, W, c)[0]) < 1e-4
    before = sched.cache.capacity
    many = [(("m", i), tokens(3 + i, seed=10 + i), [2 + i]) for i in range(before + 3)]      # more requests than slots: the cache grows
    logits = sched.step(many)
    assert sched.cache.capacity > before
    for row, (_, p, _) in enumerate(many):
        assert rel_err(logits[row:row + 1], O.forward(cfg, W, p)[0][-1:]) < 1e-4
    got = sched.step([("c", [7], [0])])                            # a request that lived through the growth goes on
    assert rel_err(got, O.forward(cfg, W, c + [7])[0][-1:]) < 1e-4


# ------------------------------------------------------------------------------------------------------------ mask edges
def sharp_cfg():
    """Large score scales make the softmax pick single keys, so a key that is wrongly seen or missed moves the logits."""
    layers = [O.window_attention_cfg(heads=2, kv_heads=1, dim=8, vdim=8, window=7, keep_first=3, scale=3.0, mlp=None),
              O.chunk_attention_cfg(heads=2, kv_heads=2, dim=8, vdim=8, chunk=6, scale=2.0, mlp=O.dense_cfg(16))]
    return O.model_cfg(layers, softcap=50.0)


@pytest.mark.parametrize("device", DEVICES)
def test_mask_edges_show_in_the_logits(device, tmp_path):
    cfg = sharp_cfg()
    W = O.random_weights(cfg, seed=4)
    W["l1.mix.q.norm"] = W["l1.mix.q.norm"] * 4.0                 # the whole-projection norm fixes the size of q: sharpen through its weight
    model, _ = make(tmp_path, cfg, device, weights=W)
    toks = tokens(40, seed=9)
    want, _ = O.forward(cfg, W, toks)
    for cuts in ([40], [22] + [1] * 18, [1] * 40, [5, 2, 9, 24]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got, want) < 2e-4, cuts
    # an implementation whose window, kept-first count or chunk is one off would be noticed
    for shift in (dict(window_shift=1), dict(window_shift=-1), dict(keep_shift=1), dict(keep_shift=-1), dict(chunk_shift=1),
                  dict(chunk_shift=-1)):
        wrong, _ = O.forward(cfg, W, toks, **shift)
        assert rel_err(wrong, want) > 20 * 2e-4, shift


@pytest.mark.parametrize("device", DEVICES)
def test_one_key_stands_out_at_every_edge(device, tmp_path):
    """One attention block; a probe token whose key matches the last query far better than any other sits just inside or just
    outside the window, the kept-first rows or the chunk — in a prompt, and with the query decoded alone."""
    for kind in ("window", "chunk"):
        if kind == "window":
            layer = O.window_attention_cfg(heads=1, kv_heads=1, dim=4, vdim=4, window=9, keep_first=2, rot=O.rot_cfg(0, 1.0), scale=6.0)
        else:
            layer = O.chunk_attention_cfg(heads=1, kv_heads=1, dim=4, vdim=4, chunk=8, rot=O.rot_cfg(0, 1.0), scale=6.0)
        layer["mixer"]["rot"] = {"dims": 0, "base": 1.0}
        cfg = O.model_cfg([layer], vocab=12, width=8, softcap=None)
        W = O.random_weights(cfg, seed=11)
        W["l0.mix.k"] = W["l0.mix.q"].clone()                     # one head, no rotation: a token's key is its own query, so the
        if kind == "chunk":                                       # probe (the same token as the last one) gets the top score
            W["l0.mix.k.norm"] = W["l0.mix.q.norm"].clone()
        model, _ = make(tmp_path, cfg, device, weights=W)
        n = 37
        # (just inside, just outside) pairs of probe positions: the kept-first rows, the window's far edge, the chunk's start
        pairs = [(1, 2), (n - 9, n - 10)] if kind == "window" else [(n - 1 - (n - 1) % 8, n - 1 - (n - 1) % 8 - 1), (32, 31)]
        last = {}
        for probe_at in sorted({p for pair in pairs for p in pair} | {0, 3, n - 8, 7, 8}):
            toks = [5] * n
            toks[probe_at] = 3
            toks[-1] = 3                                          # the last query looks for the probe's key
            want, _ = O.forward(cfg, W, toks)
            last[probe_at] = want[-1:]
            for cuts in ([n], [n - 1, 1], [n - 12] + [1] * 12):
                got, = run_schedule(model, [toks], [cuts])
                assert rel_err(got[-1:], want[-1:]) < 2e-4, (kind, probe_at, cuts)
        for inside, outside in pairs:                             # the probe matters: seeing it or not moves the last logits
            assert rel_err(last[inside], last[outside]) > 100 * 2e-4, (kind, inside, outside)


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_over_many_ring_wraps(device, tmp_path):
    cfg = mixed_cfg()
    model, W = make(tmp_path, cfg, device)
    toks = tokens(75, seed=21)
    want, _ = O.forward(cfg, W, toks)
    got, = run_schedule(model, [toks], [[4] + [1] * 71])
    assert rel_err(got, want) < 1e-4
    got2 = run_schedule(model, [toks, toks[:50]], [[4] + [1] * 71, [11] + [1] * 39])
    assert rel_err(got2[0], want) < 1e-4 and rel_err(got2[1], want[:50]) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("case", ["one_head", "window_one", "keep_beyond_window", "chunk_one", "two_readers", "wide_values",
                                  "no_rotation_left"])
def test_other_sizes(device, tmp_path, case):
    layers = {
        "one_head": [O.chunk_attention_cfg(heads=1, kv_heads=1, dim=16, vdim=2, chunk=4, mlp=O.moe_cfg(ff=3, experts=2, top=2))],
        "window_one": [O.window_attention_cfg(heads=2, kv_heads=2, dim=4, vdim=4, window=1, keep_first=1, mlp=O.dense_cfg(8))],
        "keep_beyond_window": [O.window_attention_cfg(heads=6, kv_heads=2, dim=4, vdim=4, window=2, keep_first=5, mlp=None)],
        "chunk_one": [O.chunk_attention_cfg(heads=2, kv_heads=1, dim=4, vdim=4, chunk=1, rot=O.rot_cfg(2, 7.0)),
                      O.chunk_attention_cfg(heads=2, kv_heads=1, dim=4, vdim=4, chunk=3, rot=O.rot_cfg(2, 7.0), kv_from=0,
                                            mlp=O.dense_cfg(8))],
        "two_readers": [O.chunk_attention_cfg(heads=2, kv_heads=2, dim=4, vdim=6, chunk=4, rot=O.rot_cfg(4, 9.0), mlp=O.moe_cfg(ff=4, experts=4, top=3)),
                        O.window_attention_cfg(heads=2, kv_heads=1, dim=4, vdim=4, window=3, keep_first=1, rot=O.rot_cfg(4, 9.0)),
                        O.chunk_attention_cfg(heads=4, kv_heads=2, dim=4, vdim=6, chunk=4, rot=O.rot_cfg(4, 9.0), kv_from=0),
                        O.chunk_attention_cfg(heads=2, kv_heads=2, dim=4, vdim=6, chunk=9, rot=O.rot_cfg(4, 9.0), kv_from=0,
                                              mlp=O.dense_cfg(8))],
        "wide_values": [O.window_attention_cfg(heads=2, kv_heads=1, dim=6, vdim=40, window=4, keep_first=1, rot=O.rot_cfg(6, 20.0))],
        "no_rotation_left": [O.window_attention_cfg(heads=2, kv_heads=1, dim=12, vdim=4, window=5, keep_first=0, rot=O.rot_cfg(2, 5.0))],
    }[case]
    cfg = O.model_cfg(layers, vocab=31, width=12, embedding_scale=1.0, softcap=None if case == "one_head" else 9.0)
    model, W = make(tmp_path, cfg, device, seed=7)
    toks = tokens(21, vocab=31, seed=2)
    want, _ = O.forward(cfg, W, toks)
    for cuts in ([21], [6] + [1] * 15, [2, 8, 11]):
        got, = run_schedule(model, [toks], [cuts])
        assert rel_err(got, want) < 1e-4, cuts


def test_a_block_cannot_read_the_keys_of_a_later_or_keyless_block(tmp_path):
    bad = O.model_cfg([O.chunk_attention_cfg(kv_from=1), O.chunk_attention_cfg()])
    with pytest.raises(ValueError):
        make(tmp_path, bad, "cpu", weights=O.random_weights(O.model_cfg([O.chunk_attention_cfg(), O.chunk_attention_cfg()])))


# ------------------------------------------------------------------------------------------------------------- generation
@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_entry_points(device, tmp_path):
    cfg = mixed_cfg()
    W = O.random_weights(cfg, seed=2)
    path = save_model(tmp_path, cfg, W)
    model = load_pretrained(path, dtype=torch.float32, device=device)
    prompts = [tokens(7, seed=1), tokens(12, seed=2), tokens(3, seed=3)]
    want = [O.greedy(cfg, W, p, 9) for p in prompts]
    assert RequestScheduler(model).generate(prompts, max_new_tokens=9) == want
    assert model.state_cache().live() == 0
    # the Generator protocol of the other causal LMs: a left-padded batch
    width = max(len(p) for p in prompts)
    ids = torch.tensor([[0] * (width - len(p)) + p for p in prompts], device=device)
    mask = torch.tensor([[0] * (width - len(p)) + [1] * len(p) for p in prompts], device=device)
    out = model.generate(ids, attention_mask=mask, max_length=width + 9, do_sample=False, use_cache=True, eos_token_id=None,
                         pad_token_id=0)
    assert [row[width:].tolist() for row in out] == want
    spec = importlib.util.spec_from_file_location("generate_tool", os.path.join(REPO, "tools", "generate.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    out = tool.main(["--model", path, "--prompts", ";".join(" ".join(map(str, p)) for p in prompts), "--max-new-tokens", "9",
                     "--dtype", "float32", "--device", device])
    assert out == want


@pytest.mark.parametrize("device", DEVICES)
def test_random_init_from_the_config_record(device):
    from libai_b200.config import LazyConfig, instantiate

    node = LazyConfig.load(os.path.join(REPO, "configs", "common", "models", "nefelorn.py")).model
    node.cfg.width, node.cfg.vocab = 32, 90
    for lc in node.cfg.layers:
        lc["mixer"].update(heads=2, kv_heads=1, dim=8, vdim=8)
        lc["mixer"]["rot"]["dims"] = 8
        if lc["mlp"] and lc["mlp"]["kind"] == "dense":
            lc["mlp"]["ff"] = 16
        elif lc["mlp"]:
            lc["mlp"]["expert"]["ff"] = 8
    with param_defaults(dtype=torch.float32, device=device, seed=3):
        model = instantiate(node).eval()
    out = RequestScheduler(model).generate([[1, 2, 3, 4, 5], [7]], max_new_tokens=5)
    assert [len(o) for o in out] == [5, 5] and all(0 <= t < 90 for o in out for t in o)


# ------------------------------------------------------------------------------------------------------ kernels (GPU only)
def _gpu_model(tmp_path, D, G, rep, window, keep, chunk, dtype):
    layers = [O.window_attention_cfg(heads=G * rep, kv_heads=G, dim=D, vdim=D, window=window, keep_first=keep, rot=O.rot_cfg(D // 2, 1e4),
                                     mlp=O.dense_cfg(32)),       # no experts here: in bf16 a close router call would flip a position
              O.chunk_attention_cfg(heads=G * rep, kv_heads=G, dim=D, vdim=D, chunk=chunk, rot=O.rot_cfg(D, 1e4), mlp=O.dense_cfg(64))]
    cfg = O.model_cfg(layers, vocab=64, width=64)
    return make(tmp_path, cfg, "cuda", dtype=dtype, seed=D)[0], cfg


@pytest.mark.gpu
@pytest.mark.parametrize("D,G,rep", [(32, 2, 2), (48, 1, 3), (64, 2, 4), (96, 1, 1), (128, 1, 8)])
def test_tensor_core_prompts_and_grouped_decode_match_the_generic_kernels(tmp_path, monkeypatch, D, G, rep):
    """bf16: the tensor-core prompt kernel and the grouped split kernel of single-token steps against the one-warp-per-head
    kernel, on prompts that cross many key tiles, continue from cached rows and decode past the window."""
    model, cfg = _gpu_model(tmp_path, D, G, rep, window=150, keep=5, chunk=70, dtype=torch.bfloat16)
    prompts = [tokens(n, vocab=64, seed=n) for n in (333, 64, 201)]
    cuts = [[200, 133] + [1] * 0, [64], [130, 71]]
    fast = run_schedule(model, prompts, cuts)
    dec_fast = run_schedule(model, prompts[:2], [[300] + [1] * 33, [30] + [1] * 34], cuda_graphs=False)
    monkeypatch.setattr(KF, "MMA_HEAD_SIZES", ())
    monkeypatch.setattr(KF, "GROUPED_DECODE", False)
    slow = run_schedule(model, prompts, cuts)
    dec_slow = run_schedule(model, prompts[:2], [[300] + [1] * 33, [30] + [1] * 34], cuda_graphs=False)
    for a, b in zip(fast + dec_fast, slow + dec_slow):
        assert rel_err(a, b.float().cpu()) < 2e-2
    # and the fp32 kernels, grouped and not, agree to rounding
    model32, _ = _gpu_model(tmp_path, D, G, rep, window=150, keep=5, chunk=70, dtype=torch.float32)
    one = run_schedule(model32, prompts[:1], [[300] + [1] * 33], cuda_graphs=False)
    monkeypatch.setattr(KF, "GROUPED_DECODE", True)
    two = run_schedule(model32, prompts[:1], [[300] + [1] * 33], cuda_graphs=False)
    assert rel_err(one[0], two[0].cpu()) < 1e-5
    assert rel_err(one[0], slow[0][:333].float().cpu()) < 5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("T", [17, 300, 1500])
@torch.no_grad()
def test_grouped_expert_products_in_bf16(T):
    """bf16 prompts: experts as two launches of the grouped GEMM over rows sorted by expert (ranges padded to 128 rows, one
    expert without any token, one with several row blocks) against the pair-by-pair kernels and the float64 oracle."""
    width, ff, experts, top, scale = 64, 32, 7, 2, 1.3
    cfg = O.model_cfg([O.chunk_attention_cfg(mlp=O.moe_cfg(ff, experts, top, scale))], width=width)
    W = O.random_weights(cfg, seed=5)
    W["l0.mlp.router"][3] = -W["l0.mlp.router"][0] * 4.0 - 1.0      # rarely, if ever, chosen
    W["l0.mlp.router"][0] = W["l0.mlp.router"][0] * 4.0             # chosen by about half of the tokens
    with param_defaults(dtype=torch.bfloat16, device="cuda"):
        moe = MoEFeedForward(width, ff, experts, top, router_scale=scale)
        ident = DynamicTanh(width)
    moe.router.copy_(W["l0.mlp.router"])
    moe.gate_up.copy_(torch.stack([torch.cat([W[f"l0.mlp.e{e}.gate"], W[f"l0.mlp.e{e}.up"]]) for e in range(experts)]))
    moe.down.copy_(torch.stack([W[f"l0.mlp.e{e}.down"] for e in range(experts)]))
    ident.alpha.fill_(2.0 ** -10)                                   # tanh(a v) / a ≈ v
    ident.weight.fill_(2.0 ** 10)
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(T)).to(torch.bfloat16)
    pairs, _, _ = moe(h.cuda(), graph_safe=True)
    ys, pos, cw = moe(h.cuda())
    assert pos is not None and ys.shape[0] % 128 == 0
    x = torch.zeros(T, width, device="cuda")
    KF.dyt_residual(x, ys, post=ident.triple(), pos=pos, cw=cw)
    assert rel_err(x, pairs.cpu()) < 2e-2                           # both round to bf16, at different places
    want = torch.stack([O.moe_ff(h[t].double(), W, "l0.", cfg["layers"][0]["mlp"]["router"]) for t in range(min(T, 40))])
    assert rel_err(x[:40], want) < 2e-2 and rel_err(pairs[:40], want) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("width,vocab", [(20, 37), (36, 101)])
def test_sizes_the_fast_paths_refuse_in_bf16(tmp_path, width, vocab):
    """bf16 with a width, a vocabulary, head and expert sizes that are no multiples of 8: every product and kernel falls back to
    its general form and the result stays within bf16 rounding of the oracle."""
    layers = [O.chunk_attention_cfg(heads=3, kv_heads=1, dim=6, vdim=10, chunk=9, rot=O.rot_cfg(4, 40.0), mlp=O.moe_cfg(ff=6, experts=5, top=2)),
              O.window_attention_cfg(heads=2, kv_heads=2, dim=10, vdim=6, window=7, keep_first=3, rot=O.rot_cfg(10, 40.0), mlp=O.dense_cfg(12)),
              O.chunk_attention_cfg(heads=6, kv_heads=1, dim=6, vdim=10, chunk=5, rot=O.rot_cfg(4, 40.0), kv_from=0, mlp=O.dense_cfg(20))]
    cfg = O.model_cfg(layers, vocab=vocab, width=width)
    W = O.random_weights(cfg, seed=width)
    model, _ = make(tmp_path, cfg, "cuda", dtype=torch.bfloat16, weights=W)
    prompts = [tokens(n, vocab=vocab, seed=n) for n in (33, 18)]
    want = [O.forward(cfg, W, p)[0] for p in prompts]
    got = run_schedule(model, prompts, [[20] + [1] * 13, [18]])
    errs = [rel_err(g, w) for g, w in zip(got, want)]
    assert max(errs) < 8e-2, errs                                  # (a close router call may move single positions)
    assert float(torch.median(torch.tensor([rel_err(got[0][i:i + 1], want[0][i:i + 1]) for i in range(33)]))) < 2e-2


@pytest.mark.gpu
def test_serving_precision_and_graphed_steps(tmp_path):
    cfg = mixed_cfg(width=32)
    W = O.random_weights(cfg, seed=3)
    path = save_model(tmp_path, cfg, W)
    model = load_pretrained(path, dtype=torch.bfloat16, device="cuda")
    prompts = [tokens(n, seed=n) for n in (24, 9, 40)]
    want = [O.forward(cfg, W, p)[0] for p in prompts]
    cuts = [[10] + [1] * 14, [5] + [1] * 4, [25] + [1] * 15]
    eager = run_schedule(model, prompts, cuts, cuda_graphs=False)
    graphed = run_schedule(model, prompts, cuts, cuda_graphs=True)
    for e, g_, w in zip(eager, graphed, want):
        assert rel_err(e, w) < 5e-2
        assert rel_err(g_, e.float().cpu()) < 1e-6              # a replayed step computes exactly what an eager one does
