"""Bumodra against a plain float64 oracle (``bumodra_oracle.py``): every mechanism alone, whole prompts, decoding through the
state cache, prompt portions, ragged batches, slot reuse, window edges, far keys, long decoding, odd sizes, generation.

The CPU parametrisation exercises the framework's PyTorch operators; the ``cuda`` one (marked ``gpu``) the sm_100a kernels.
"""
import json
import math
import os

import pytest
import torch

from libai_b200.inference.ragged import RaggedBatch
from libai_b200.inference.scheduler import RequestScheduler
from libai_b200.inference.state_cache import SequenceStateCache
from libai_b200.layers import GatedDeltaMixer, LatentAttention, RMSLayerNorm
from libai_b200.layers._param import param_defaults
from libai_b200.models.utils.model_loader.auto import load_pretrained
from libai_b200.ops import seq_functional as SF

from . import bumodra_oracle as O

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]
_PARAM_TO_CKPT = {"q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "dq_norm": "dq.norm", "dkv_norm": "dkv.norm"}


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


def make(tmp_path, cfg, device, dtype=torch.float32, seed=0):
    weights = O.random_weights(cfg, seed)
    return load_pretrained(save_model(tmp_path, cfg, weights), dtype=dtype, device=device), weights


def run_schedule(model, prompts, cuts):
    """Feed ``prompts`` together: step s brings ``cuts[i][s]`` tokens of prompt i (requests that have nothing left drop out).
    Returns per prompt the logits of all its positions."""
    sched = RequestScheduler(model)
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
            got[i].append(logits[o:o + n])
            o += n
        sched.finish([("r", i) for i, p in enumerate(prompts) if at[i] == len(p)])
    assert sched.cache.live() == 0
    return [torch.cat(g) for g in got]


def mixed_cfg(**kw):
    layers = [O.delta_cfg(heads=2, kv_heads=2, dim=8, vdim=8, conv=2), O.attention_cfg(window=6),
              O.delta_cfg(channel=True, heads=4, kv_heads=2, dim=12, vdim=8, conv=4), O.delta_cfg(heads=3, kv_heads=1, ff=0)]
    return O.model_cfg(layers, loop={"start": 1, "stop": 3, "times": 2}, **kw)


def tokens(n, vocab=50, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------------------ mechanisms alone
def _fill(module, weights, prefix):
    with torch.no_grad():
        for name, p in module.named_parameters():
            p.copy_(weights[prefix + _PARAM_TO_CKPT.get(name, name)].to(p.dtype))


def _one_sequence(device, n, past=0):
    return RaggedBatch([n], [1], [past], device)


@pytest.mark.parametrize("device", DEVICES)
def test_zero_centred_norm_and_embedding_gather(device):
    g = torch.Generator().manual_seed(1)
    table, w = torch.randn(11, 20, generator=g), 0.3 * torch.randn(20, generator=g)
    ids = torch.tensor([3, 3, 10, 0])
    with param_defaults(dtype=torch.float32, device=device):
        norm = RMSLayerNorm(20, eps=1e-4, zero_centered=True)
    with torch.no_grad():
        norm.weight.copy_(w)
    out = torch.empty(4, 20, device=device)
    norm.rows(table.to(device), out, ids=ids.to(device))
    assert torch.allclose(out.cpu().double(), O.zero_centred_norm(table[ids].double(), w.double(), 1e-4), atol=1e-5)
    assert not torch.allclose(out.cpu().double(), O.plain_norm(table[ids].double(), w.double(), 1e-4), atol=1e-2)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_in_portions(device, taps):
    g = torch.Generator().manual_seed(taps)
    C, T = 7, 13
    x, w = torch.randn(T, C, generator=g), torch.randn(C, taps, generator=g)
    want = O.short_conv_silu(x.double(), w.double())
    tail = torch.full((3, taps - 1, C), 7.0, device=device)      # dirty slot: must be ignored when past == 0
    got, at = [], 0
    for n in (1, 2, 5, 1, 4):
        out = torch.empty(n, C, device=device)
        SF.short_conv(x[at:at + n].to(device), w.to(device), tail, _one_sequence(device, n, at), out)
        got.append(out.cpu())
        at += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("channel,heads,kv_heads,dim,vdim", [(False, 4, 2, 8, 12), (True, 3, 3, 12, 8), (False, 2, 1, 40, 72),
                                                              (True, 1, 1, 5, 3)])
def test_delta_mixer_alone(device, channel, heads, kv_heads, dim, vdim):
    lc = O.delta_cfg(channel=channel, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=3, ff=0)
    cfg = O.model_cfg([lc], width=16)
    w = O.random_weights(cfg, seed=3)
    with param_defaults(dtype=torch.float32, device=device):
        mix = GatedDeltaMixer(16, heads, kv_heads, dim, vdim, 3, decay="channel" if channel else "head", decay_rank=6,
                              gate="sigmoid_lowrank" if channel else "silu", gate_rank=5, eps=1e-5)
    _fill(mix, w, "l0.mix.")
    cache = SequenceStateCache(device, torch.float32)
    bufs = _state(cache, mix)
    for b in bufs.values():
        b.fill_(3.0)                                             # a reused slot is dirty
    h = torch.randn(21, 16, generator=torch.Generator().manual_seed(4))
    want = O.delta_mixer(h.double(), {k: v.double() for k, v in w.items()}, "l0.mix.", lc["mixer"], 1e-5, channel)
    whole = mix(h.to(device), _one_sequence(device, 21), bufs)
    assert torch.allclose(whole.cpu().double(), want, atol=2e-5, rtol=1e-4)
    parts, at = [], 0
    for n in (17, 1, 1, 2):                                      # a prompt, two single tokens, a portion of two
        parts.append(mix(h[at:at + n].to(device), _one_sequence(device, n, at), bufs).cpu())
        at += n
    assert torch.allclose(torch.cat(parts).double(), want, atol=2e-5, rtol=1e-4)


def _state(cache, mixer):
    kind, shape = mixer.state_spec()
    return cache.buffers(cache.register(kind, **shape))


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("window,dim,vdim,kv_rank", [(5, 8, 12, 9), (1, 4, 4, 6), (64, 16, 8, 40), (7, 24, 40, 33)])
def test_latent_attention_alone(device, window, dim, vdim, kv_rank):
    lc = O.attention_cfg(heads=3, dim=dim, vdim=vdim, q_rank=10, kv_rank=kv_rank, window=window, scale=1.5, ff=0)
    w = O.random_weights(O.model_cfg([lc], width=16), seed=5)
    with param_defaults(dtype=torch.float32, device=device):
        att = LatentAttention(16, 3, dim, vdim, 10, kv_rank, window, scale=1.5, eps=1e-5)
    _fill(att, w, "l0.mix.")
    cache = SequenceStateCache(device, torch.float32)
    bufs = _state(cache, att)
    bufs["ring"].fill_(9.0)
    T = 40
    h = torch.randn(T, 16, generator=torch.Generator().manual_seed(6))
    wd = {k: v.double() for k, v in w.items()}
    want = O.latent_attention(h.double(), wd, "l0.mix.", lc["mixer"], 1e-5)
    assert torch.allclose(att(h.to(device), _one_sequence(device, T), bufs).cpu().double(), want, atol=2e-5, rtol=1e-4)
    parts, at = [], 0
    for n in [3, 2] + [1] * 20 + [9, 2, 4]:                      # portions and single tokens across several windows
        parts.append(att(h[at:at + n].to(device), _one_sequence(device, n, at), bufs).cpu())
        at += n
    assert at == T and torch.allclose(torch.cat(parts).double(), want, atol=2e-5, rtol=1e-4)
    if 1 < window < T:                                           # the test can tell a window that is one token off
        for other in (window - 1, window + 1):
            off = O.latent_attention(h.double(), wd, "l0.mix.", lc["mixer"], 1e-5, window=other)
            assert (off - want).abs().max() > 1e-2


@pytest.mark.parametrize("device", DEVICES)
def test_absorbed_single_token_form_equals_expanded_form(device):
    lc = O.attention_cfg(heads=2, dim=8, vdim=8, q_rank=8, kv_rank=16, window=4, ff=0)
    w = O.random_weights(O.model_cfg([lc], width=16), seed=8)
    outs = []
    for absorbed in (True, False):
        with param_defaults(dtype=torch.float32, device=device):
            att = LatentAttention(16, 2, 8, 8, 8, 16, 4, eps=1e-5, absorbed_decode=absorbed)
        _fill(att, w, "l0.mix.")
        cache = SequenceStateCache(device, torch.float32)
        bufs = _state(cache, att)
        h = torch.randn(12, 16, generator=torch.Generator().manual_seed(9)).to(device)
        outs.append(torch.cat([att(h[t:t + 1], _one_sequence(device, 1, t), bufs) for t in range(12)]).cpu())
    assert torch.allclose(outs[0], outs[1], atol=1e-5)


# ---------------------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("device", DEVICES)
def test_whole_prompt_and_every_block_run(device, tmp_path):
    cfg = mixed_cfg()
    model, w = make(tmp_path, cfg, device)
    toks = tokens(19)
    want, stream = O.model_logits(cfg, w, toks, return_stream=True)
    taps = []
    cache = model.state_cache()
    slot = cache.allocate(1)
    got = model.step(torch.tensor(toks, device=device), RaggedBatch([19], slot, [0], device), tap=lambda r, x: taps.append(x.cpu().clone()))
    cache.free(slot)
    assert len(taps) == len(O.block_runs(cfg)) == 6
    for r, x in enumerate(taps):
        assert torch.allclose(x.double(), stream[r], atol=1e-4, rtol=1e-4), f"block run {r}"
    assert rel_err(got, want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_decoding_and_portions_equal_the_whole_prompt(device, tmp_path):
    cfg = mixed_cfg()
    model, w = make(tmp_path, cfg, device)
    toks = tokens(31, seed=2)
    want = O.model_logits(cfg, w, toks)
    for cuts in ([31], [1] * 31, [20] + [1] * 11, [2, 2, 3, 5, 2, 7, 1, 9], [6, 25], [29, 2]):
        got = run_schedule(model, [toks], [cuts])[0]
        assert rel_err(got, want) < 1e-4, cuts


@pytest.mark.parametrize("device", DEVICES)
def test_ragged_batches_equal_each_request_alone(device, tmp_path):
    cfg = mixed_cfg()
    model, w = make(tmp_path, cfg, device)
    prompts = [tokens(n, seed=10 + n) for n in (1, 23, 9, 14)]
    want = [O.model_logits(cfg, w, p) for p in prompts]
    # all start together with different lengths, then go on one token at a time; the short ones leave first
    cuts = [[1], [12] + [1] * 11, [5] + [1] * 4, [3] + [1] * 11]
    for got, ref in zip(run_schedule(model, prompts, cuts), want):
        assert rel_err(got, ref) < 1e-4
    alone = [run_schedule(model, [p], [c])[0] for p, c in zip(prompts, cuts)]
    for a, b in zip(run_schedule(model, prompts, cuts), alone):
        assert torch.allclose(a, b, atol=1e-4)


@pytest.mark.parametrize("device", DEVICES)
def test_slots_are_reused_and_the_cache_grows(device, tmp_path):
    cfg = mixed_cfg()
    model, w = make(tmp_path, cfg, device)
    sched = RequestScheduler(model)
    first = tokens(17, seed=40)
    sched.step([("a", first, [])])
    slot = sched.slot_of["a"]
    sched.finish(["a"])
    other = tokens(11, seed=41)
    got = sched.step([("b", other, list(range(11)))])
    assert sched.slot_of["b"] == slot                            # the freed slot, still holding the first request's state
    assert rel_err(got, O.model_logits(cfg, w, other)) < 1e-4
    many = [tokens(4 + i, seed=50 + i) for i in range(9)]        # more live requests than the cache started with
    got = sched.step([(("m", i), p, [len(p) - 1]) for i, p in enumerate(many)])
    assert sched.cache.capacity >= 10
    got2 = sched.step([("b", [7], [0])])                         # the older request survived the growth
    assert rel_err(got2, O.model_logits(cfg, w, other + [7])[-1:]) < 1e-4
    for i, p in enumerate(many):
        assert rel_err(got[i:i + 1], O.model_logits(cfg, w, p)[-1:]) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_window_edges_in_prompts_and_in_decoding(device, tmp_path):
    # sharp softmax (large scale): a key that is wrongly seen or missed at the window's edge changes the logits visibly
    layers = [O.attention_cfg(heads=2, dim=8, vdim=8, q_rank=8, kv_rank=8, window=5, scale=2.5, ff=0),
              O.attention_cfg(heads=2, dim=8, vdim=8, q_rank=8, kv_rank=8, window=3, scale=2.5)]
    cfg = O.model_cfg(layers)
    model, w = make(tmp_path, cfg, device)
    toks = tokens(26, seed=5)
    want = O.model_logits(cfg, w, toks)
    shifted = json.loads(json.dumps(cfg))
    shifted["layers"][0]["mixer"]["mask"]["size"] = 6
    assert rel_err(O.model_logits(shifted, w, toks), want) > 1e-2
    for cuts in ([26], [4] + [1] * 22, [5] + [1] * 21, [6] + [1] * 20, [3, 3, 2, 18], [1] * 26):
        assert rel_err(run_schedule(model, [toks], [cuts])[0], want) < 1e-4, cuts


@pytest.mark.parametrize("device", DEVICES)
def test_far_tokens_reach_the_end_through_the_recurrent_state(device, tmp_path):
    cfg = O.model_cfg([O.delta_cfg(heads=2, kv_heads=1, dim=8, vdim=8, conv=2), O.delta_cfg(channel=True, heads=2, kv_heads=2, ff=0)])
    weights = O.random_weights(cfg, seed=7)
    weights["l0.mix.A_log"].fill_(-9.0)                          # decay ≈ 1: the state keeps what the first tokens wrote
    weights["l1.mix.A_log"].fill_(-9.0)
    model = load_pretrained(save_model(tmp_path, cfg, weights), dtype=torch.float32, device=device)
    toks = tokens(150, seed=6)
    want = O.model_logits(cfg, weights, toks)
    changed = O.model_logits(cfg, weights, [(toks[0] + 1) % 50] + toks[1:])
    assert rel_err(changed[-1:], want[-1:]) > 1e-3               # the last position does depend on the first token
    assert rel_err(run_schedule(model, [toks], [[150]])[0], want) < 1e-4
    assert rel_err(run_schedule(model, [toks], [[30] + [1] * 120])[0], want) < 1e-4     # long decoding


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("variant", ["no_loop", "loop_of_one_pass", "loop_over_everything", "single_heads"])
def test_other_layouts(device, tmp_path, variant):
    if variant == "no_loop":
        cfg = O.model_cfg([O.attention_cfg(window=40), O.delta_cfg(ff=0)], width=16, vocab=33)
    elif variant == "loop_of_one_pass":
        cfg = O.model_cfg([O.delta_cfg(channel=True, conv=2), O.attention_cfg(window=2, ff=0)], loop={"start": 1, "stop": 2, "times": 1})
    elif variant == "loop_over_everything":
        cfg = O.model_cfg([O.attention_cfg(window=4), O.delta_cfg(conv=5)], width=40, loop={"start": 0, "stop": 2, "times": 3})
    else:
        cfg = O.model_cfg([O.attention_cfg(heads=1, dim=4, vdim=6, q_rank=3, kv_rank=5, window=3),
                           O.delta_cfg(heads=1, kv_heads=1, dim=6, vdim=4, conv=2)], width=8, vocab=9)
    model, w = make(tmp_path, cfg, device, seed=11)
    toks = tokens(15, vocab=cfg["vocab"], seed=12)
    want = O.model_logits(cfg, w, toks)
    assert rel_err(run_schedule(model, [toks], [[15]])[0], want) < 1e-4
    assert rel_err(run_schedule(model, [toks], [[7] + [1] * 8])[0], want) < 1e-4


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_generate_and_the_scheduler(device, tmp_path):
    cfg = mixed_cfg()
    cfg.update(pad_token_id=0, eos_token_id=None)
    model, w = make(tmp_path, cfg, device)
    prompts = [tokens(6, seed=20), tokens(3, seed=21)]
    prompts = [[t or 1 for t in p] for p in prompts]             # 0 is the padding token
    want = [O.greedy(cfg, w, p, 5) for p in prompts]
    sched = RequestScheduler(model)
    assert sched.generate(prompts, max_new_tokens=5) == want
    assert sched.cache.live() == 0
    ids = torch.tensor([prompts[0], [0] * 3 + prompts[1]])       # left padded, as Generator.generate expects
    out = model.generate(ids, max_new_tokens=5, pad_token_id=0)
    assert out[0, 6:].tolist() == want[0] and out[1, 6:].tolist() == want[1]
    assert model.state_cache().live() == 0
    again = model.generate(ids, max_new_tokens=5, pad_token_id=0, use_cache=False)
    assert torch.equal(out, again)
    torch.manual_seed(0)
    sampled = model.generate(ids[:1], max_new_tokens=4, do_sample=True, top_k=5, temperature=0.7)
    assert sampled.shape == (1, 10)


@pytest.mark.gpu
def test_bfloat16_serving_precision_stays_near_the_oracle(tmp_path):
    cfg = mixed_cfg(width=64)
    model, w = make(tmp_path, cfg, "cuda", dtype=torch.bfloat16)
    toks = tokens(48, seed=30)
    want = O.model_logits(cfg, w, toks)
    whole = run_schedule(model, [toks], [[48]])[0]
    split = run_schedule(model, [toks], [[40] + [1] * 8])[0]
    assert rel_err(whole, want) < 0.08 and rel_err(split, want) < 0.08
    from libai_b200 import ops

    assert ops.launch_count() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("D,V,window", [(64, 64, 40), (32, 64, 1), (128, 128, 200), (64, 32, 64), (128, 64, 7)])
def test_tensor_core_window_attention_equals_the_generic_kernel(D, V, window):
    g = torch.Generator().manual_seed(D + V + window)
    H, lens, past = 3, [70, 1, 129, 5], [0, 300, 17, 64]
    cache_rows = min(max(past), window - 1) + 1
    rb = RaggedBatch(lens, [0, 1, 2, 3], past, "cuda")
    T, E = rb.tokens, rb.ext(window).rows
    q = torch.randn(T, H * D, generator=g).to("cuda", torch.bfloat16)
    kv = torch.randn(E, H * (D + V), generator=g).to("cuda", torch.bfloat16)
    gate = torch.randn(T, H, generator=g).to("cuda", torch.bfloat16)
    a, b = torch.empty(T, H * V, dtype=torch.bfloat16, device="cuda"), torch.empty(T, H * V, dtype=torch.bfloat16, device="cuda")
    SF.window_attention(q, kv, gate, rb, a, H, D, V, window, 0.2, mma=True)
    SF.window_attention(q, kv, gate, rb, b, H, D, V, window, 0.2, mma=False)
    assert cache_rows >= 1 and torch.isfinite(a.float()).all()
    assert (a.float() - b.float()).abs().max() < 0.03


@pytest.mark.parametrize("device", DEVICES)
def test_long_window_single_token_steps(device):
    # a window of more than 64 positions takes the split single-token kernel on the GPU (partial softmax per 32 positions)
    lc = O.attention_cfg(heads=5, dim=8, vdim=8, q_rank=8, kv_rank=24, window=70, scale=1.0, ff=0)
    w = O.random_weights(O.model_cfg([lc], width=16), seed=13)
    with param_defaults(dtype=torch.float32, device=device):
        att = LatentAttention(16, 5, 8, 8, 8, 24, 70, scale=1.0, eps=1e-5)
    _fill(att, w, "l0.mix.")
    bufs = _state(SequenceStateCache(device, torch.float32), att)
    T = 110
    h = torch.randn(T, 16, generator=torch.Generator().manual_seed(14))
    want = O.latent_attention(h.double(), {k: v.double() for k, v in w.items()}, "l0.mix.", lc["mixer"], 1e-5)
    parts = [att(h[:3].to(device), _one_sequence(device, 3), bufs).cpu()]
    parts += [att(h[t:t + 1].to(device), _one_sequence(device, 1, t), bufs).cpu() for t in range(3, T)]
    assert torch.allclose(torch.cat(parts).double(), want, atol=2e-5, rtol=1e-4)


def test_command_line_generation_and_lazy_config(tmp_path, capsys):
    import importlib.util

    from libai_b200.config import LazyConfig, instantiate

    cfg = mixed_cfg()
    weights = O.random_weights(cfg, seed=2)
    folder = save_model(tmp_path, cfg, weights)
    spec = importlib.util.spec_from_file_location("generate_tool", os.path.join(os.path.dirname(__file__), "..", "..", "tools", "generate.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    out = tool.main(["--model", folder, "--prompts", "5 17 3;9 9 12 40 2", "--max-new-tokens", "4", "--dtype", "float32", "--device", "cpu"])
    assert out == [O.greedy(cfg, weights, [5, 17, 3], 4), O.greedy(cfg, weights, [9, 9, 12, 40, 2], 4)]
    assert len(capsys.readouterr().out.strip().splitlines()) == 2
    node = LazyConfig.load(os.path.join(os.path.dirname(__file__), "..", "..", "configs", "common", "models", "bumodra.py")).model
    node.cfg.width, node.cfg.vocab = 64, 100
    for lc in node.cfg.layers:
        lc["mlp"]["ff"] = 32
        lc["mixer"].update(heads=2, dim=8, vdim=8)
        if "kv_heads" in lc["mixer"]:
            lc["mixer"]["kv_heads"] = 2 if lc["type"] == "channel_delta" else 1
        for k in ("q_rank", "kv_rank", "decay_rank", "gate_rank"):
            if k in lc["mixer"]:
                lc["mixer"][k] = 8
    with param_defaults(dtype=torch.float32, device="cpu"):
        model = instantiate(node).eval()
    ids = torch.randint(3, 100, (2, 7))
    a = model.generate(ids, max_new_tokens=3)
    assert a.shape == (2, 10) and torch.equal(a, model.generate(ids, max_new_tokens=3, use_cache=False))


@pytest.mark.gpu
@pytest.mark.parametrize("act", [SF.ACT_COPY, SF.ACT_RELU2, SF.ACT_SILU, SF.ACT_GELU_TANH])
def test_slice_activation_between_column_slices(act):
    x = torch.randn(37, 96, device="cuda").to(torch.bfloat16)
    wide = torch.zeros(37, 128, dtype=torch.bfloat16, device="cuda")
    SF.slice_act(x[:, 16:80], wide[:, 32:96], act)               # 16-byte path: offsets and widths are multiples of 8
    odd = torch.zeros(37, 50, dtype=torch.bfloat16, device="cuda")
    SF.slice_act(x[:, 3:40], odd[:, 5:42], act)                  # element path
    v = x.float()
    want = {SF.ACT_COPY: v, SF.ACT_RELU2: torch.relu(v) ** 2, SF.ACT_SILU: torch.nn.functional.silu(v),
            SF.ACT_GELU_TANH: torch.nn.functional.gelu(v, approximate="tanh")}[act]
    assert torch.allclose(wide[:, 32:96].float(), want[:, 16:80], atol=2e-2, rtol=2e-2)
    assert torch.allclose(odd[:, 5:42].float(), want[:, 3:40], atol=2e-2, rtol=2e-2)
    assert float(wide[:, :32].abs().max()) == 0 and float(wide[:, 96:].abs().max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("C,taps", [(64, 4), (24, 2), (20, 3)])
def test_short_convolution_bf16_ragged_batch_on_the_gpu(C, taps):
    g = torch.Generator().manual_seed(C + taps)
    lens, past = [9, 1, 2, 14], [0, 5, 1, 0]
    rb = RaggedBatch(lens, [3, 0, 2, 1], past, "cuda")
    x = torch.randn(sum(lens), C, generator=g).to(torch.bfloat16)
    w = torch.randn(C, taps, generator=g).to(torch.bfloat16)
    tail = torch.randn(4, taps - 1, C, generator=g).to(torch.bfloat16)
    out_gpu = torch.empty(sum(lens), C, dtype=torch.bfloat16, device="cuda")
    tail_gpu = tail.cuda()
    SF.short_conv(x.cuda(), w.cuda(), tail_gpu, rb, out_gpu)
    out_cpu, tail_cpu = torch.empty(sum(lens), C, dtype=torch.bfloat16), tail.clone()
    SF.short_conv(x, w, tail_cpu, RaggedBatch(lens, [3, 0, 2, 1], past, "cpu"), out_cpu)
    assert torch.allclose(out_gpu.cpu().float(), out_cpu.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(tail_gpu.cpu(), tail_cpu)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_single_token_steps_from_cuda_graphs_equal_eager_steps(tmp_path, dtype):
    cfg = mixed_cfg(width=32)
    model, w = make(tmp_path, cfg, "cuda", dtype=dtype)
    prompts = [tokens(n, seed=60 + n) for n in (9, 4, 13)]
    tails = [tokens(14, seed=70), tokens(6, seed=71), tokens(14, seed=72)]        # the second request leaves the batch early

    def run(graphs):
        sched = RequestScheduler(model, cuda_graphs=graphs)
        out = [sched.step([(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])]
        for t in range(14):
            live = [i for i in range(3) if t < len(tails[i])]
            out.append(sched.step([(i, [tails[i][t]], [0]) for i in live]))
            sched.finish([i for i in live if t + 1 == len(tails[i])])
        assert sched.cache.live() == 0
        return torch.cat(out), sched

    eager, _ = run(False)
    graphed, sched = run(True)
    assert any(v != "seen" for v in sched._graphs.values())                        # graphs were captured and replayed
    assert torch.allclose(eager, graphed, atol=1e-5 if dtype == torch.float32 else 2e-2)
    if dtype == torch.float32:
        want = O.model_logits(cfg, w, prompts[0] + tails[0])[len(prompts[0]) - 1:]
        got = torch.stack([graphed[0]] + [graphed[3 + (3 * t if t < 6 else 18 + 2 * (t - 6))] for t in range(14)])
        assert rel_err(got, want) < 1e-4
