"""Pefivik on the engine against the plain oracle (oracle/pefivik_oracle.py): every mechanism alone, prompts in one piece, in
portions down to two tokens and token by token, batched decode steps of unequal requests, slots that are freed and used
again, keys far away and at the edges of key tiles and key splits, a sink that dominates, gates that forget nothing or
everything, the first tokens of a sequence, long decoding, greedy generation through generate() and the continuous batcher.
Small configurations whose sizes differ from one another (and from multiples of the kernels' tiles), random weights, both
number formats; where random weights would hide a fault the weights are shaped so that it shows."""
import copy
import threading

import numpy as np
import pytest
import torch

from oracle import pefivik_oracle as O

pytestmark = pytest.mark.gpu

LAT = {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "vdim": 16, "kv_rank": 40, "scale": 0.25}}
LAT_ODD = {"type": "latent_attention", "mixer": {"heads": 5, "dim": 9, "vdim": 7, "kv_rank": 21, "scale": 0.4}}      # nothing a multiple of 4
LAT_ONE = {"type": "latent_attention", "mixer": {"heads": 1, "dim": 16, "vdim": 16, "kv_rank": 16, "scale": 1.0}}
LAT_MANY = {"type": "latent_attention", "mixer": {"heads": 40, "dim": 8, "vdim": 4, "kv_rank": 24, "scale": 0.3}}    # more heads than a CTA's pairs
LAT_WIDE = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "vdim": 48, "kv_rank": 288, "scale": 0.15}}  # latent wider than 256
HG = {"type": "hgrn2", "mixer": {"heads": 3, "dim": 20, "vdim": 24}}
HG_ODD = {"type": "hgrn2", "mixer": {"heads": 1, "dim": 17, "vdim": 10}}        # one key slice partly empty
HG_BIG = {"type": "hgrn2", "mixer": {"heads": 2, "dim": 40, "vdim": 70}}        # three blocks of value columns
DENSE = {"kind": "dense", "ff": 72}
DENSE_ODD = {"kind": "dense", "ff": 50}
MOE = {"kind": "moe", "expert": {"ff": 24}, "shared": {"ff": 40},
       "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}, "scale": 1.7}}
MOE_ONE = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 1, "groups": {"count": 1, "keep": 1}, "scale": 1.0}}   # no shared expert
MOE_SINGLES = {"kind": "moe", "expert": {"ff": 16}, "shared": {"ff": 8},
               "router": {"experts": 4, "top": 3, "groups": {"count": 4, "keep": 3}, "scale": 0.5}}                                    # groups of one expert


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def config(layers, width=72, vocab=150, eps=1e-5, loop=None, bigram=(61, 7, 13), mult=0.6, softcap=15.0):
    cfg = {"architecture": "Pefivik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult, "layers": copy.deepcopy(layers),
           "embedding": {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


CFG_MAIN = config([layer(LAT, DENSE), layer(HG, MOE), layer(LAT, MOE), layer(HG, None)], loop=(1, 3, 3))
# one bucket (every bigram hashes to row 0), multiplier 1, no soft-cap, a "loop" of one pass (its vector is still added), odd sizes
CFG_ODD = config([layer(HG_ODD, DENSE_ODD), layer(LAT_ODD, MOE_ONE)], width=50, vocab=77, eps=1e-3, bigram=(1, 1, 1), mult=1.0, softcap=None,
                 loop=(1, 2, 1))
# the loop covers every layer; big hash multipliers
CFG_LOOP_ALL = config([layer(LAT_ONE, MOE_SINGLES), layer(HG_BIG, DENSE)], width=64, loop=(0, 2, 2), bigram=(521, 1000003, 999983), mult=0.9)
CFG_TAIL_LOOP = config([layer(HG, None), layer(LAT_MANY, DENSE_ODD)], width=48, loop=(1, 2, 2), mult=0.5)


def build(cfg, dtype=torch.float32, seed=0, weights=None, **limits):
    from llava.model import PefivikConfig, PefivikForCausalLM

    w = weights if weights is not None else O.random_weights(cfg, seed=seed)
    limits = {"max_batch": 4, "max_seq": 256, **limits}
    model = PefivikForCausalLM(PefivikConfig(**cfg), {k: torch.from_numpy(np.asarray(v, np.float32)).bfloat16() for k, v in w.items()}, dtype=dtype, **limits)
    return model, w


def tokens_for(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def row_errors(a, b):
    a = torch.as_tensor(np.asarray(a.detach().cpu() if torch.is_tensor(a) else a), dtype=torch.float64)
    b = torch.as_tensor(np.asarray(b.detach().cpu() if torch.is_tensor(b) else b), dtype=torch.float64)
    return ((a - b) ** 2).mean(-1).sqrt() / (b.std(-1) + 1e-12)


def err(a, b):
    """rms difference over std of the reference, per row, worst row"""
    return float(row_errors(a, b).max())


def close(a, b, dtype, tight=False):
    """fp32: every row within rounding. bf16: nine rows in ten within the format's rounding (a router choice between two
    nearly equal scores may fall the other way for a row when its input is rounded to bf16)."""
    e = row_errors(a, b).flatten()
    if dtype == torch.float32:
        return float(e.max()) < (2e-5 if tight else 2e-4)
    return float(torch.quantile(e, 0.9)) < (2e-2 if tight else 6e-2)


def run_schedule(eng, kv, slot, toks, cuts, decode_single=True):
    """Feed toks in portions of the sizes `cuts` (the rest one by one); a single token of a running request takes the decode
    step when decode_single, else the portion call. Returns logits of every position."""
    out, at, first = [], 0, True
    sizes = list(cuts) + [1] * (len(toks) - sum(cuts))
    for n in sizes:
        part = toks[at:at + n]
        if n == 1 and not first and decode_single:
            out.append(eng.decode_step(kv, torch.tensor(part, dtype=torch.int32), slot0=slot))
        else:
            out.append(eng.append_tokens(kv, slot, part, list(range(n)), restart=first))
        at, first = at + n, False
    return torch.cat(out)


def one_layer(cfg_layer, **kw):
    return config([cfg_layer], loop=None, softcap=None, **kw)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["latent", "latent_odd", "latent_one_head", "latent_many_heads", "latent_wide", "hgrn2", "hgrn2_odd", "hgrn2_big",
                                  "dense", "dense_odd", "moe", "moe_top1", "moe_single_groups"])
def test_each_mechanism_alone(name, dtype):
    """One layer: the residual stream after it equals x + m * mechanism(norm(x)) of the oracle's function for that mechanism."""
    mixers = {"latent": LAT, "latent_odd": LAT_ODD, "latent_one_head": LAT_ONE, "latent_many_heads": LAT_MANY, "latent_wide": LAT_WIDE, "hgrn2": HG,
              "hgrn2_odd": HG_ODD, "hgrn2_big": HG_BIG}
    mlps = {"dense": DENSE, "dense_odd": DENSE_ODD, "moe": MOE, "moe_top1": MOE_ONE, "moe_single_groups": MOE_SINGLES}
    lay = layer(mixers.get(name, HG_ODD), mlps.get(name))
    cfg = one_layer(lay, width=50 if name.endswith("odd") else 72)
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 37)
    _, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = O.embedding(cfg, w, toks)
    h = O.scalar_rms_norm(x, w["l0.norm1"], eps)
    mixer = O.latent_attention if lay["type"] == "latent_attention" else O.hgrn2
    x = x + m * mixer(h, O.layer_params(w, 0, "mix"), lay["mixer"], eps)
    if lay["mlp"]:
        h = O.scalar_rms_norm(x, w["l0.norm2"], eps)
        p = O.layer_params(w, 0, "mlp")
        x = x + m * (O.dense_ff(h, p, eps) if lay["mlp"]["kind"] == "dense" else O.moe_ff(h, p, lay["mlp"]))
    assert close(hidden[0, 0], x, dtype)


def test_router_choices_and_weights():
    """The router alone: a model whose only routed expert output is visible (no shared expert, identity-like scale) must pick the
    oracle's experts; checked through the layer output for three group layouts, in fp32 where no choice is a close call."""
    for mlp in (MOE, MOE_ONE, MOE_SINGLES):
        cfg = one_layer(layer(HG_ODD, mlp), width=40)
        w = O.random_weights(cfg, seed=4)
        model, _ = build(cfg, torch.float32, weights=w)
        toks = tokens_for(cfg, 90, seed=2)
        _, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
        _, stream = O.forward(cfg, w, toks)
        assert err(hidden[0, 0], stream[0]) < 2e-4
        model.invalidate_engine()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [CFG_MAIN, CFG_ODD, CFG_LOOP_ALL, CFG_TAIL_LOOP], ids=["main", "odd", "loop_all", "loop_tail"])
def test_whole_prompt_against_the_oracle(cfg, dtype):
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 70)
    logits, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    ref, stream = O.forward(cfg, w, toks)
    assert hidden.shape[1] == len(O.layer_runs(cfg)) == stream.shape[0]
    for i in range(stream.shape[0]):
        assert close(hidden[0, i], stream[i], dtype), f"residual stream after layer run {i}"
    assert close(logits[0], ref, dtype)
    if dtype == torch.float32:
        assert err(logits[0, :3], ref[:3]) < 2e-4, "first tokens of a sequence"
        single = model.forward(torch.tensor([toks[:1]]))
        assert err(single[0], ref[:1]) < 2e-4, "a prompt of one token"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [CFG_MAIN, CFG_ODD, CFG_LOOP_ALL], ids=["main", "odd", "loop_all"])
def test_portions_and_token_by_token_equal_the_whole_prompt(cfg, dtype):
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(4, 256)
    toks = tokens_for(cfg, 61, seed=3)
    whole = run_schedule(eng, kv, 0, toks, [len(toks)])
    ref, _ = O.forward(cfg, w, toks)
    assert close(whole, ref, dtype)
    schedules = {"token by token": [1], "twos": [2] * 30, "mixed": [7, 2, 1, 13, 2, 2, 5, 1, 3], "one then all": [1, 60], "all but one": [60],
                 "nines": [9] * 6}
    for name, cuts in schedules.items():
        for decode_single in (True, False):
            got = run_schedule(eng, kv, 1 + decode_single, toks, cuts, decode_single)
            assert close(got, whole, dtype, tight=True), f"{name} (decode step for single tokens: {decode_single})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_keeps_cache_and_state(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 150, seed=5)
    got = run_schedule(eng, kv, 0, toks, [8])          # 142 decode steps
    ref, _ = O.forward(cfg, w, toks)
    assert close(got[-40:], ref[-40:], dtype)
    assert close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_decode_of_unequal_requests_equals_each_alone(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype, max_batch=6)
    eng = model._ensure_engine()
    kv = eng.new_kv(6, 256)
    reqs = [tokens_for(cfg, n, seed=10 + n) for n in (37, 14, 21, 50, 13)]
    steps = 12
    alone = [run_schedule(eng, kv, 5, r, [len(r) - steps]) for r in reqs]      # slot 5, one request after the other
    for b, r in enumerate(reqs):
        eng.append_tokens(kv, b, r[:len(r) - steps], [], restart=True)
    got = [[] for _ in reqs]
    for s in range(steps):                                                    # one decode step over the five slots
        col = torch.tensor([r[len(r) - steps + s] for r in reqs], dtype=torch.int32)
        lg = eng.decode_step(kv, col)
        for b in range(len(reqs)):
            got[b].append(lg[b])
    for b, r in enumerate(reqs):
        assert close(torch.stack(got[b]), alone[b][-steps:], dtype, tight=True), f"request {b}"
    ref, _ = O.forward(cfg, w, reqs[1])
    assert close(torch.stack(got[1]), ref[-steps:], dtype)


def test_a_slot_that_is_freed_and_used_again_starts_clean():
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    a, b = tokens_for(cfg, 90, seed=21), tokens_for(cfg, 33, seed=22)
    fresh = run_schedule(eng, kv, 1, b, [20])
    run_schedule(eng, kv, 0, a, [50])                      # leaves latent rows, recurrent state and a carried token behind
    kv.free_slot(0)
    assert kv.lengths(2)[0] == 0
    again = run_schedule(eng, kv, 0, b, [20])
    assert err(again, fresh) < 1e-6
    third = run_schedule(eng, kv, 0, b, [2, 2])            # restart on a slot that was not freed, shortest portions
    assert err(third, fresh) < 2e-5
    with pytest.raises(ValueError):
        eng.append_tokens(kv, 0, [0] * 300, [], restart=False)   # beyond the slot's capacity


def sharp_latent_model(T, seed=7, heads=2, rank=36):
    """One latent-attention layer whose queries are scaled up until the softmax is almost an argmax: for most positions ONE
    key, anywhere in the past, carries the output, so a key that is dropped or seen twice (the edge of a key tile of 32,
    of a key split, of a portion) moves the result by far more than the tolerance."""
    lay = layer({"type": "latent_attention", "mixer": {"heads": heads, "dim": 16, "vdim": 12, "kv_rank": rank, "scale": 1.0}}, None)
    cfg = one_layer(lay, width=48, vocab=400)
    w = O.random_weights(cfg, seed=seed)
    w["l0.mix.q"] = O.bf16_round(w["l0.mix.q"] * 12.0)
    w["l0.mix.sink"] = O.bf16_round(np.full(heads, -20.0))
    return cfg, w


def test_far_keys_and_tile_edges_in_prompts_portions_and_decoding():
    T = 420
    cfg, w = sharp_latent_model(T)
    toks = tokens_for(cfg, T, seed=9)
    ref, _ = O.forward(cfg, w, toks)
    # the test's premise: winners lie far back and next to multiples of 32 for many queries
    h = O.scalar_rms_norm(O.embedding(cfg, w, toks), w["l0.norm1"], cfg["norm"]["eps"])
    p = O.layer_params(w, 0, "mix")
    c = O.unit_rms(h @ p["dkv"].T, cfg["norm"]["eps"]) * p["dkv.norm"]
    s = (h @ p["q"].T)[:, :16] @ (c @ p["uk"].T)[:, :16].T
    win = np.array([int(np.argmax(s[i, :i + 1])) for i in range(T)])
    dist = np.arange(T) - win
    assert (dist > 200).sum() >= 20 and ((win % 32 == 31) | (win % 32 == 0)).sum() >= 10
    model, _ = build(cfg, torch.float32, weights=w, max_batch=2, max_seq=1024, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 1024)
    assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4, "whole prompt"
    assert err(run_schedule(eng, kv, 1, toks, [31, 2, 33, 64, 1, 95, 2, 2, 130]), ref) < 2e-4, "portions that end at and around tile edges, then decode steps"
    assert err(run_schedule(eng, kv, 0, toks, [300]), ref) < 2e-4, "120 decode steps over split keys"


def test_experts_on_tensor_cores_equal_the_plain_products(monkeypatch):
    """Long bf16 prompt portions sort their (token, choice) pairs by expert into 128-row tiles for ONE grouped tensor-core
    product per projection; short ones and fp32 use plain grouped products. Uneven expert loads, experts without tokens."""
    mlp = {"kind": "moe", "expert": {"ff": 40}, "shared": {"ff": 32},
           "router": {"experts": 10, "top": 3, "groups": {"count": 5, "keep": 3}, "scale": 1.3}}
    cfg = one_layer(layer(HG_ODD, mlp), width=64)
    w = O.random_weights(cfg, seed=6)
    w["l0.mlp.router"][7] = 0.0                       # experts that are (almost) never chosen
    w["l0.mlp.router"][2] = O.bf16_round(w["l0.mlp.router"][2] * 3.0)
    model, _ = build(cfg, torch.bfloat16, weights=w, max_seq=512, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 512)
    toks = tokens_for(cfg, 330, seed=23)
    ref, _ = O.forward(cfg, w, toks)
    got = {}
    for name, flag in (("tensor cores", "1"), ("plain", "0")):
        monkeypatch.setenv("B2_SEQ_TC", flag)
        got[name] = run_schedule(eng, kv, 0, toks, [200, 65, 64])
        assert close(got[name], ref, torch.bfloat16), name
    assert close(got["tensor cores"], got["plain"], torch.bfloat16, tight=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_absorbed_and_per_head_attention_agree(dtype, monkeypatch):
    """Long prompt portions make per-head keys and values from the cached latent rows; short ones and decode steps carry the
    query into the latent space instead. Both forms, forced on the same prompt and portions, give the same logits."""
    cfg = config([layer(LAT, None), layer(LAT_WIDE, DENSE), layer(LAT_MANY, None)], loop=(0, 2, 2))
    model, w = build(cfg, dtype, max_seq=512, max_rows=160)     # fewer workspace rows than positions: the keys are made in pieces
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 512)
    toks = tokens_for(cfg, 300, seed=19)
    ref, _ = O.forward(cfg, w, toks)
    got = {}
    for name, rows in (("per head", "1"), ("absorbed", "100000")):
        monkeypatch.setenv("B2_LATENT_MATERIALISE_ROWS", rows)
        got[name] = run_schedule(eng, kv, 0, toks, [150, 3, 120, 20])
        assert close(got[name], ref, dtype), name
    assert close(got["per head"], got["absorbed"], dtype, tight=True)


def test_a_sink_that_dominates_and_one_that_vanishes():
    """Head 0's sink is far above every score (its output all but disappears), head 1's far below (plain softmax): leaving the
    sink out, scaling it, or counting it once per key split shows in either head."""
    lay = layer(LAT, None)
    lay["mixer"]["heads"] = 2
    cfg = one_layer(lay)
    w = O.random_weights(cfg, seed=3)
    T = 200
    toks = tokens_for(cfg, T, seed=13)
    for sinks in ([6.0, -30.0], [0.5, 2.0]):
        w["l0.mix.sink"] = O.bf16_round(np.array(sinks))
        ref, stream = O.forward(cfg, w, toks)
        model, _ = build(cfg, torch.float32, weights=w, max_seq=1024)
        eng = model._ensure_engine()
        kv = eng.new_kv(2, 1024)
        assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4
        assert err(run_schedule(eng, kv, 1, toks, [150]), ref) < 2e-4, "decode steps merge key splits: the sink counts once"
        model.invalidate_engine()
    w0 = dict(w)
    w0["l0.mix.sink"] = O.bf16_round(np.array([-30.0, -30.0]))
    assert err(O.forward(cfg, w0, toks)[0], ref) > 1e-2, "premise: the sink matters for these weights"


def test_gates_that_keep_everything_or_nothing():
    """Lower bounds next to 1 keep the first tokens in the state over hundreds of steps; lower bounds of 0 with a strongly
    negative gate bias forget at once. Both ends, in a prompt, in portions of two and in decode steps."""
    lay = layer(HG, None)
    cfg = one_layer(lay, width=48)
    w = O.random_weights(cfg, seed=5)
    n = lay["mixer"]["heads"] * lay["mixer"]["dim"]
    low = np.zeros(n)
    low[::2] = 0.998
    w["l0.mix.lower"] = O.bf16_round(low)
    fb = np.zeros(n)
    fb[1::4] = -9.0
    fb[3::4] = 9.0
    w["l0.mix.f.b"] = O.bf16_round(fb)
    T = 260
    toks = tokens_for(cfg, T, seed=15)
    ref, _ = O.forward(cfg, w, toks)
    model, _ = build(cfg, torch.float32, weights=w, max_seq=512, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 512)
    assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 1, toks, [2] * 60 + [17, 16, 15]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [100]), ref) < 2e-4
    # premise: forgetting the carried state at a portion's start would show at the end of the prompt
    tail, _ = O.forward(cfg, w, toks[130:])
    assert err(tail[-20:], ref[-20:]) > 1e-2


def test_the_bigram_row_follows_the_previous_token_across_calls():
    """The hashed row depends on the token in front, which for a call's first token was fed by an earlier call (or by a decode
    step, or is absent at a sequence start)."""
    cfg = one_layer(layer(HG_ODD, None), width=40, vocab=300, bigram=(257, 29, 23))
    w = O.random_weights(cfg, seed=8)
    w["bigram"] = O.bf16_round(w["bigram"] * 4.0)
    toks = tokens_for(cfg, 40, seed=17)
    ref, _ = O.forward(cfg, w, toks)
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(3, 64)
    assert err(run_schedule(eng, kv, 0, toks, [40]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 1, toks, [1, 2, 3, 2]), ref) < 2e-4
    other = tokens_for(cfg, 25, seed=18)
    run_schedule(eng, kv, 2, other, [25])                  # slot 2 now carries another request's last token
    kv.free_slot(2)
    assert err(run_schedule(eng, kv, 2, toks, [5, 5]), ref) < 2e-4
    rows = O.bigram_rows(toks, 257, 29, 23)
    assert rows[0] == 257 and len(set(rows)) > 30


def greedy_matches_oracle(cfg, w, prompt, new_tokens, tol_margin=1e-3):
    """The generated ids, fed to the oracle, are its own greedy choices wherever its top-2 margin is not a rounding matter."""
    seq = list(prompt) + list(new_tokens)
    ref = torch.from_numpy(O.forward(cfg, w, seq)[0])
    for i, t in enumerate(new_tokens):
        row = ref[len(prompt) - 1 + i]
        top = torch.topk(row, 2)
        if float(top.values[0] - top.values[1]) > tol_margin * float(row.std()):
            assert int(top.indices[0]) == int(t), f"token {i}"


def test_greedy_generation_through_generate():
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    prompts = torch.tensor([tokens_for(cfg, 12, seed=51), tokens_for(cfg, 12, seed=52)])
    out = model.generate(prompts, max_new_tokens=10)
    assert out.shape == (2, 22) and torch.equal(out[:, :12], prompts)
    for b in range(2):
        greedy_matches_oracle(cfg, w, prompts[b].tolist(), out[b, 12:].tolist())
    solo = model.generate(prompts[1:2], max_new_tokens=10)
    assert torch.equal(solo[0], out[1])


def test_continuous_batching_of_unequal_requests():
    """Six generate() threads on three slots: requests join and leave between steps, slots are reused, and every request gets
    the ids it gets alone."""
    cfg = copy.deepcopy(CFG_MAIN)
    model, w = build(cfg, torch.float32)
    prompts = [torch.tensor([tokens_for(cfg, n, seed=60 + n)]) for n in (5, 19, 9, 30, 3, 14)]
    new = [6, 14, 9, 4, 12, 8]
    solo = [model.generate(p, max_new_tokens=n) for p, n in zip(prompts, new)]
    model.invalidate_engine()
    model.config.raw["b2_continuous_batching"] = 3
    results, errors = [None] * len(prompts), []

    def work(i):
        try:
            results[i] = model.generate(prompts[i], max_new_tokens=new[i])
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    stats = model._batcher.stats
    for i in range(len(prompts)):
        assert torch.equal(results[i], solo[i]), f"request {i}"
    assert stats["admitted"] == 6 and stats["max_active"] <= 3 and stats["rows_stepped"] > stats["steps"]
    greedy_matches_oracle(cfg, w, prompts[1][0].tolist(), results[1][0, 19:].tolist())
    model.invalidate_engine()


def test_sampled_generation_repeats_with_the_seed_and_rejects_bad_input():
    cfg = CFG_ODD
    model, _ = build(cfg, torch.bfloat16)
    p = torch.tensor([tokens_for(cfg, 8, seed=71)])
    torch.manual_seed(5)
    a = model.generate(p, do_sample=True, temperature=0.9, top_k=20, top_p=0.95, max_new_tokens=12)
    torch.manual_seed(5)
    b = model.generate(p, do_sample=True, temperature=0.9, top_k=20, top_p=0.95, max_new_tokens=12)
    assert torch.equal(a, b) and int(a.max()) < cfg["vocab"]
    with pytest.raises(ValueError):
        model.generate(torch.tensor([[cfg["vocab"] + 3, 1, 2]]), max_new_tokens=2)
    with pytest.raises(ValueError):
        model.generate(p, max_new_tokens=4000)
