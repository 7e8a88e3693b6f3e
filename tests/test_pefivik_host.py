"""CPU checks around Pefivik: the registry and configuration reader, and properties of the plain oracle that the GPU tests
rely on (causality, layer runs of a looped block, group-limited routing, the sink, gates at their bounds)."""
import json
import math

import numpy as np

from oracle import pefivik_oracle as O

LAT = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 6, "kv_rank": 12, "scale": 0.5}}
HG = {"type": "hgrn2", "mixer": {"heads": 2, "dim": 6, "vdim": 10}}
MOE = {"kind": "moe", "expert": {"ff": 8}, "shared": {"ff": 12}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}, "scale": 2.0}}
CFG = {"architecture": "Pefivik", "width": 32, "vocab": 50, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "logit_softcap": 12.0,
       "embedding": {"bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 3}}, "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [dict(LAT, mlp={"kind": "dense", "ff": 40}), dict(HG, mlp=MOE), dict(LAT, mlp=None), dict(HG, mlp={"kind": "dense", "ff": 24})]}


def test_registry_and_configuration_reader(tmp_path):
    from llava._b2 import BLOCK_PRE_RMS1, FF_MOE, FF_POLYNORM, MIXER_HGRN2, MIXER_LATENT_ATTN
    from llava.model import MODEL_REGISTRY, PefivikConfig, model_class_for

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert "Pefivik" in MODEL_REGISTRY and model_class_for(str(tmp_path)).__name__ == "PefivikForCausalLM"
    c = PefivikConfig.from_pretrained(str(tmp_path))
    md = c.model_desc()
    assert md["block"] == BLOCK_PRE_RMS1 and md["bigram_buckets"] == 37 and (md["loop_start"], md["loop_stop"], md["loop_times"]) == (1, 3, 2)
    assert abs(md["residual_mult"] - 0.8) < 1e-9 and md["logit_softcap"] == 12.0
    d = c.layer_descs({})
    assert [x["type"] for x in d] == [MIXER_LATENT_ATTN, MIXER_HGRN2, MIXER_LATENT_ATTN, MIXER_HGRN2]
    assert d[0]["ff_kind"] == FF_POLYNORM and d[0]["ff"] == 40 and d[0]["la_rank"] == 12 and d[2]["ff"] == 0
    assert d[1]["ff_kind"] == FF_MOE and (d[1]["moe_experts"], d[1]["moe_top"], d[1]["moe_groups"], d[1]["moe_keep"], d[1]["moe_shared_ff"]) == (6, 2, 3, 2, 12)
    plain = dict(CFG)
    del plain["loop"], plain["logit_softcap"]
    md = PefivikConfig(**plain).model_desc()
    assert "loop_times" not in md and md["logit_softcap"] == 0.0


def test_layer_runs_of_a_looped_block():
    assert O.layer_runs(CFG) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert O.layer_runs(dict(CFG, loop={"start": 0, "stop": 4, "times": 1})) == [(0, 0), (1, None), (2, None), (3, None)]
    no_loop = {k: v for k, v in CFG.items() if k != "loop"}
    assert O.layer_runs(no_loop) == [(i, None) for i in range(4)]


def test_oracle_is_causal_and_softcapped():
    w = O.random_weights(CFG, seed=1)
    a = list(range(3, 23))
    b = a[:12] + [49 - t for t in a[12:]]
    la, sa = O.forward(CFG, w, a)
    lb, _ = O.forward(CFG, w, b)
    assert np.allclose(la[:12], lb[:12]) and not np.allclose(la[12:], lb[12:])
    assert sa.shape == (6, 20, 32) and np.abs(la).max() < 12.0
    assert O.bigram_rows([4, 9, 9], 37, 5, 3) == [37, (4 * 5 + 9 * 3) % 37, (9 * 5 + 9 * 3) % 37]


def test_group_limited_routing():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}, "scale": 3.0}
    logits = np.array([[4.0, -9.0, 1.0, 1.1, 3.0, -9.0]])        # group sums: s(4)+s(-9) < s(1)+s(1.1) : the best single expert is shut out
    chosen, weights = O.route(logits, np.eye(6), r)
    assert sorted(chosen[0]) == [2, 3]
    s = 1 / (1 + np.exp(-np.array([1.1, 1.0])))
    assert np.allclose(sorted(weights[0], reverse=True), s / s.sum() * 3.0)
    chosen, _ = O.route(logits, np.eye(6), dict(r, groups={"count": 3, "keep": 3}))
    assert sorted(chosen[0]) == [0, 4]


def test_polynorm_sink_and_gate_bounds():
    z = np.array([[1.0, -2.0, 3.0, 0.5]])
    n = lambda u: u / math.sqrt(float((u * u).mean()) + 1e-6)  # noqa: E731
    want = 0.5 * n(z[0]) + 0.25 * n(z[0] ** 2) - 0.1 * n(z[0] ** 3) + 0.3
    assert np.allclose(O.polynorm(z, [0.5, 0.25, -0.1, 0.3], 1e-6)[0], want)
    cfg = {**CFG, "layers": [dict(LAT, mlp=None)]}
    cfg.pop("loop")
    w = O.random_weights(cfg, seed=2)
    h = np.random.default_rng(0).standard_normal((9, 32))
    p = O.layer_params(w, 0, "mix")
    plain = O.latent_attention(h, dict(p, sink=np.array([-40.0, -40.0])), LAT["mixer"], 1e-5)
    drowned = O.latent_attention(h, dict(p, sink=np.array([40.0, 40.0])), LAT["mixer"], 1e-5)
    assert np.abs(drowned).max() < 1e-9 * max(1.0, np.abs(plain).max()) + 1e-12 and np.abs(plain).max() > 1e-3
    cfg = {**cfg, "layers": [dict(HG, mlp=None)]}
    w = O.random_weights(cfg, seed=3)
    p = O.layer_params(w, 0, "mix")
    frozen = O.hgrn2(h, dict(p, lower=np.ones(12)), HG["mixer"], 1e-5)      # f = 1: nothing is ever written
    assert np.abs(frozen).max() == 0.0
    p0 = dict(p, lower=np.zeros(12))
    p0["f.b"] = np.full(12, -60.0)                                           # f = 0: the state is the current token alone
    memoryless = O.hgrn2(h, p0, HG["mixer"], 1e-5)
    assert np.allclose(memoryless[5:6], O.hgrn2(h[5:6], p0, HG["mixer"], 1e-5))
