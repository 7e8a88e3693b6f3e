"""Katadra on the engine against the plain oracle (oracle/katadra_oracle.py): every mechanism alone, prompts in one piece,
in portions and token by token, batched decode steps, slots that are reused, distance-bias buckets and temperature steps at
their edges, long decoding, greedy generation through generate() and the continuous batcher. Small configurations with
sizes that differ from one another (and from multiples of the kernels' tiles), random weights, both number formats."""
import copy
import threading

import pytest
import torch

from oracle import katadra_oracle as O

pytestmark = pytest.mark.gpu

MAMBA = {"type": "mamba2", "mixer": {"heads": 4, "vdim": 24, "state": 20, "groups": 2, "conv": 3, "norm_groups": 4}, "mlp": None}
PAR = {"type": "parallel", "mlp": {"kind": "dense", "ff": 136},
       "mixer": {"left": {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "bias_max": 40, "scale": 0.3, "softcap": 8.0,
                          "q_temp": {"coef": 0.7, "every": 5}, "rel_rows": 10},
                 "right": {"heads": 3, "dim": 24, "decay_rank": 5}, "left_scale": 0.8, "right_scale": 1.3}}
# odd sizes: nothing is a multiple of 4, one key slice is partly empty (dim 17 > 16), one group, kv_heads == heads, every == 1
MAMBA_ODD = {"type": "mamba2", "mixer": {"heads": 3, "vdim": 10, "state": 7, "groups": 1, "conv": 2, "norm_groups": 1},
             "mlp": {"kind": "dense", "ff": 50}}
PAR_ODD = {"type": "parallel", "mlp": None,
           "mixer": {"left": {"heads": 4, "kv_heads": 4, "dim": 9, "vdim": 7, "bias_max": 12, "scale": 1.0, "softcap": 3.0,
                              "q_temp": {"coef": 0.25, "every": 1}, "rel_rows": 7},
                     "right": {"heads": 2, "dim": 17, "decay_rank": 3}, "left_scale": 1.0, "right_scale": 0.5}}


def borrow(layer, j):
    out = copy.deepcopy(layer)
    out["weights_of"] = j
    return out


def config(layers, width=96, vocab=160, eps=1e-5):
    return {"architecture": "Katadra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


MAMBA5 = {"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 36, "groups": 4, "conv": 5, "norm_groups": 2}, "mlp": None}
CFG_MAIN = config([MAMBA, PAR, borrow(MAMBA, 0), borrow(PAR, 1)])
CFG_FWD = config([borrow(MAMBA5, 2), PAR, MAMBA5], width=64)       # the first layer computes with the LAST layer's tensors
CFG_ODD = config([PAR_ODD, MAMBA_ODD, MAMBA_ODD], width=90, vocab=77, eps=1e-3)


def build(cfg, dtype=torch.float32, seed=0, weights=None, **limits):
    from llava.model import KatadraConfig, KatadraForCausalLM

    w = weights if weights is not None else O.random_weights(cfg, seed=seed)
    limits = {"max_batch": 4, "max_seq": 256, **limits}
    model = KatadraForCausalLM(KatadraConfig(**cfg), {k: v.bfloat16() for k, v in w.items()}, dtype=dtype, **limits)
    return model, w


def tokens_for(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def err(a, b):
    """rms difference over std of the reference, per row, worst row"""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((((a - b) ** 2).mean(-1).sqrt() / (b.std(-1) + 1e-12)).max())


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["mamba2", "attention", "rwkv", "mamba2_odd", "attention_odd", "rwkv_odd", "feed_forward"])
def test_each_mechanism_alone(name, dtype):
    """One layer, one mixer: the residual stream after it equals embed + LayerNorm(mechanism(embed)) of the oracle."""
    base = {"mamba2": MAMBA, "mamba2_odd": MAMBA_ODD, "feed_forward": MAMBA_ODD}.get(name)
    odd = name.endswith("_odd")
    if base is None:
        base = copy.deepcopy(PAR_ODD if odd else PAR)
        left = name.startswith("attention")
        base["mixer"]["left_scale"], base["mixer"]["right_scale"] = (1.0, 0.0) if left else (0.0, 1.0)
    layer = copy.deepcopy(base)
    if name != "feed_forward":
        layer["mlp"] = None
    cfg = config([layer], width=90 if odd else 96)
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 29)
    _, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    x0 = w["embed"][torch.tensor(toks)].double()
    wd = {k: v.double() for k, v in w.items()}
    mix = {k[7:]: v for k, v in wd.items() if k.startswith("l0.mix.")}
    eps = cfg["norm"]["eps"]
    if layer["type"] == "mamba2":
        m = O.mamba2_mixer(x0, mix, layer["mixer"], eps)
    elif name.startswith("attention"):
        m = O.attention_left(x0, {k[5:]: v for k, v in mix.items() if k.startswith("left.")}, layer["mixer"]["left"], eps)
    else:
        m = O.rwkv_right(x0, {k[6:]: v for k, v in mix.items() if k.startswith("right.")}, layer["mixer"]["right"], eps)
    x1 = x0 + O.layer_norm(m, wd["l0.norm1"], wd["l0.norm1.b"], eps)
    if name == "feed_forward":
        f = O.feed_forward(x1, {"up": wd["l0.mlp.up"], "down": wd["l0.mlp.down"]})
        x1 = x1 + O.layer_norm(f, wd["l0.norm2"], wd["l0.norm2.b"], eps)
    assert err(hidden[0, 0], x1) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [CFG_MAIN, CFG_ODD, CFG_FWD], ids=["main", "odd", "borrow_forward"])
def test_whole_prompt_against_the_oracle(cfg, dtype):
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 70)
    logits, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    ref, layers = O.forward(cfg, w, toks, return_layers=True)
    for i in range(len(cfg["layers"])):
        assert err(hidden[0, i], layers[i]) < TOL[dtype], f"residual stream after layer {i}"
    assert err(logits[0], ref) < TOL[dtype]
    assert err(logits[0, :3], ref[:3]) < TOL[dtype], "first tokens of a sequence"


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [CFG_MAIN, CFG_ODD], ids=["main", "odd"])
def test_portions_and_token_by_token_equal_the_whole_prompt(cfg, dtype):
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(4, 256)
    toks = tokens_for(cfg, 61, seed=3)
    whole = run_schedule(eng, kv, 0, toks, [len(toks)])
    ref = O.forward(cfg, w, toks)
    assert err(whole, ref) < TOL[dtype]
    tight = 2e-5 if dtype == torch.float32 else 2e-2   # the same arithmetic in another order / through other kernels
    schedules = {"token by token": [1], "twos": [2] * 30, "mixed": [7, 2, 1, 13, 2, 2, 5, 1, 3], "one then all": [1, 60],
                 "all but one": [60]}
    for name, cuts in schedules.items():
        for decode_single in (True, False):
            got = run_schedule(eng, kv, 1 + decode_single, toks, cuts, decode_single)
            assert err(got, whole) < tight, f"{name} (decode step for single tokens: {decode_single})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_keeps_the_state(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 120, seed=5)
    got = run_schedule(eng, kv, 0, toks, [8])          # 112 decode steps
    ref = O.forward(cfg, w, toks)
    assert err(got[-40:], ref[-40:]) < TOL[dtype]
    assert err(got, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_decode_of_unequal_requests_equals_each_alone(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype, max_batch=6)
    eng = model._ensure_engine()
    kv = eng.new_kv(6, 256)
    reqs = [tokens_for(cfg, n, seed=10 + n) for n in (37, 14, 21, 50, 13)]    # five rows: the step's Linears take the tile GEMM in bf16
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
    tight = 2e-5 if dtype == torch.float32 else 2e-2
    for b, r in enumerate(reqs):
        assert err(torch.stack(got[b]), alone[b][-steps:]) < tight, f"request {b}"
    ref = O.forward(cfg, w, reqs[1])
    assert err(torch.stack(got[1]), ref[-steps:]) < TOL[dtype]


def test_a_slot_that_is_freed_and_used_again_starts_clean():
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    a, b = tokens_for(cfg, 90, seed=21), tokens_for(cfg, 33, seed=22)
    fresh = run_schedule(eng, kv, 1, b, [20])
    run_schedule(eng, kv, 0, a, [50])                      # leaves state, convolution tails and 90 key/value rows behind
    kv.free_slot(0)
    assert kv.lengths(2)[0] == 0
    again = run_schedule(eng, kv, 0, b, [20])
    assert err(again, fresh) < 1e-6
    with pytest.raises(ValueError):
        eng.append_tokens(kv, 0, [0] * 300, [], restart=False)   # beyond the slot's capacity


def test_distance_buckets_and_temperature_steps_at_their_edges():
    """The bias table gets values that make ONE bucket win the softmax by far, so a key that lands in the wrong bucket (one
    token off at an edge, a far key treated as near) moves the output visibly; the temperature period is short, so the
    steps of floor((p + 1) / every) fall inside the prompt. Checked in a prompt, in portions and in decode steps."""
    layer = copy.deepcopy(PAR)
    layer["mlp"] = None
    layer["mixer"]["left_scale"], layer["mixer"]["right_scale"] = 1.0, 0.0
    layer["mixer"]["left"].update(rel_rows=10, bias_max=40, q_temp={"coef": 2.0, "every": 7})
    cfg = config([layer])
    T = 64
    toks = tokens_for(cfg, T, seed=31)
    rows, H = 10, layer["mixer"]["left"]["heads"]
    for winner in (4, 5, 7, 9):                              # last exact row, first logarithmic row, a middle row, the far row
        w = O.random_weights(cfg, seed=2)
        rel = torch.full((rows, H), -12.0)
        rel[winner] = 6.0
        w["l0.mix.left.rel"] = rel
        ref = O.forward(cfg, w, toks)
        model, _ = build(cfg, torch.float32, weights=w)
        eng = model._ensure_engine()
        kv = eng.new_kv(2, 128)
        assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4, f"prompt, bucket {winner}"
        assert err(run_schedule(eng, kv, 1, toks, [9, 2, 30]), ref) < 2e-4, f"portions + decode steps, bucket {winner}"
        model.invalidate_engine()
    edges = [n for n in range(1, 80) if O.distance_bucket(n, rows, 40) != O.distance_bucket(n - 1, rows, 40)]
    assert edges[:5] == [1, 2, 3, 4, 5] and max(edges) <= 40 and O.distance_bucket(39, rows, 40) == 9 - (O.distance_bucket(39, rows, 40) != 9)


def test_decode_attention_with_split_keys_equals_the_prompt_path():
    """A decode step cuts long contexts into key ranges that are merged afterwards; the prompt path never does."""
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32, max_batch=2, max_seq=1024)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 1024)
    toks = tokens_for(cfg, 700, seed=41)
    whole = eng.append_tokens(kv, 0, toks, list(range(690, 700)), restart=True)
    eng.append_tokens(kv, 1, toks[:690], [], restart=True)
    dec = torch.cat([eng.decode_step(kv, torch.tensor([t], dtype=torch.int32), slot0=1) for t in toks[690:]])
    assert err(dec, whole) < 2e-5


def greedy_matches_oracle(cfg, w, prompt, new_tokens, tol_margin=1e-3):
    """The generated ids, fed to the oracle, are its own greedy choices wherever its top-2 margin is not a rounding matter."""
    seq = list(prompt) + list(new_tokens)
    ref = O.forward(cfg, w, seq)
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
