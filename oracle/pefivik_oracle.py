"""Plain restatement of the Pefivik decoder, one function per mechanism, in float64, token by token, without any cache.

Nothing here is shared with the engine: the tests compare the engine's kernels, caches and schedules with these loops.
A model is (cfg, w): `cfg` the dictionary of config.json, `w` a dictionary name -> numpy array with the checkpoint's names
(`embed`, `bigram`, `loop.step`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`).

Notation: h is a sublayer's input [T, width]; every Linear weight is [out, in] and applied as h @ W.T.
"""
import math

import numpy as np

F = np.float64


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---------------------------------------------------------------------------------------------------------------- embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every position: hash of (previous, current); the first token takes the extra last row."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embedding(cfg, w, tokens):
    x = w["embed"].astype(F)[list(tokens)]
    bg = cfg.get("embedding", {}).get("bigram")
    if bg:
        x = x + w["bigram"].astype(F)[bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))]
    return x


# ---------------------------------------------------------------------------------------------------------------- norms
def scalar_rms_norm(x, g, eps):
    """Unit RMS times ONE learned number."""
    return unit_rms(x, eps) * float(np.asarray(g, F).reshape(-1)[0])


# ---------------------------------------------------------------------------------------------------------------- mixers
def latent_attention(h, p, mix, eps):
    """Causal attention whose keys and values are both read off a low-rank latent c_j = rms(W_dkv h_j) * g; no positions;
    the softmax denominator holds one extra term exp(sink_head); each head's output is gated by sigmoid(W_g h)."""
    T = h.shape[0]
    H, dk, dv = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
    scale = float(mix["scale"])
    q = (h @ p["q"].T).reshape(T, H, dk)
    c = unit_rms(h @ p["dkv"].T, eps) * p["dkv.norm"]
    k = (c @ p["uk"].T).reshape(T, H, dk)
    v = (c @ p["uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ p["g"].T)                      # [T, H]
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        for hd in range(H):
            s = (k[: i + 1, hd] @ q[i, hd]) * scale   # [i+1]
            sink = float(p["sink"][hd])
            m = max(s.max(), sink)
            e = np.exp(s - m)
            den = e.sum() + math.exp(sink - m)
            out[i, hd] = (e[:, None] * v[: i + 1, hd]).sum(0) / den * gate[i, hd]
    return out.reshape(T, H * dv) @ p["o"].T


def hgrn2(h, p, mix, eps):
    """Gated linear recurrence: per head S <- diag(f) S + (1 - f) v^T, o = S^T q, with q = silu(W_q h) and the forget gate
    f = l + (1 - l) sigmoid(W_f h + b) bounded below by l; per-head unit RMS of o with a weight shared by the heads."""
    T = h.shape[0]
    H, dk, dv = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
    q = silu(h @ p["q"].T).reshape(T, H, dk)
    v = (h @ p["v"].T).reshape(T, H, dv)
    low = p["lower"].reshape(H, dk)
    f = low + (1.0 - low) * sigmoid(h @ p["f"].T + p["f.b"]).reshape(T, H, dk)
    S = np.zeros((H, dk, dv), F)
    o = np.zeros((T, H, dv), F)
    for t in range(T):
        for hd in range(H):
            S[hd] = f[t, hd][:, None] * S[hd] + (1.0 - f[t, hd])[:, None] * v[t, hd][None, :]
            o[t, hd] = S[hd].T @ q[t, hd]
    o = unit_rms(o, eps) * p["norm"]
    return o.reshape(T, H * dv) @ p["o"].T


# ---------------------------------------------------------------------------------------------------------------- feed-forward
def polynorm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with element-wise powers and N = unit RMS over a token's vector."""
    a, b, c, e = [float(v) for v in coef]
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, p, eps):
    z = h @ p["up"].T + p["up.b"]
    return polynorm(z, p["act"], eps) @ p["down"].T + p["down.b"]


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router_w, r):
    """For every token: the chosen experts and their weights. Scores are sigmoids; experts form `count` groups of
    neighbours, a group's score is the sum of its two largest scores, only experts of the best `keep` groups compete."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = int(groups["count"]), int(groups["keep"])
    per = E // G
    s = sigmoid(h @ router_w.T)
    chosen, weights = [], []
    for t in range(h.shape[0]):
        gs = [np.sort(s[t, g * per:(g + 1) * per])[::-1][:2].sum() for g in range(G)]
        alive = sorted(range(G), key=lambda g: -gs[g])[:keep]
        cand = [e for g in alive for e in range(g * per, (g + 1) * per)]
        best = sorted(cand, key=lambda e: -s[t, e])[:top]
        sc = np.array([s[t, e] for e in best], F)
        chosen.append(best)
        weights.append(sc / (sc.sum() + 1e-20) * float(r["scale"]))
    return chosen, weights


def moe_ff(h, p, mlp):
    r = mlp["router"]
    chosen, weights = route(h, p["router"], r)
    out = np.zeros((h.shape[0], p["e0.down"].shape[0]), F)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * gated_expert(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out += gated_expert(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


# ---------------------------------------------------------------------------------------------------------------- the model
def layer_params(w, i, part):
    pre = f"l{i}.{part}."
    return {k[len(pre):]: np.asarray(v, F) for k, v in w.items() if k.startswith(pre)}


def layer_runs(cfg):
    """[(layer, pass or None)]: the pass number is given for the FIRST layer of every pass of the looped block."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["times"]) < 1 or int(loop["stop"]) <= int(loop["start"]):
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def run_layer(cfg, w, i, x):
    layer, eps, m = cfg["layers"][i], float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    h = scalar_rms_norm(x, w[f"l{i}.norm1"], eps)
    mixer = {"latent_attention": latent_attention, "hgrn2": hgrn2}[layer["type"]]
    x = x + m * mixer(h, layer_params(w, i, "mix"), layer["mixer"], eps)
    mlp = layer.get("mlp")
    if mlp:
        h = scalar_rms_norm(x, w[f"l{i}.norm2"], eps)
        p = layer_params(w, i, "mlp")
        x = x + m * (dense_ff(h, p, eps) if mlp["kind"] == "dense" else moe_ff(h, p, mlp))
    return x


def forward(cfg, w, tokens):
    """tokens -> (logits [T, vocab], residual stream after every layer run [runs, T, width])."""
    x0 = embedding(cfg, w, tokens)
    x, stream = x0.copy(), []
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + np.asarray(w["loop.step"], F)[t]
        x = run_layer(cfg, w, i, x)
        stream.append(x.copy())
    z = scalar_rms_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ np.asarray(w["head"], F).T
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * np.tanh(z / float(cap))
    return z, np.stack(stream)


# ---------------------------------------------------------------------------------------------------------------- random models
def bf16_round(a):
    """Round float32 values to the nearest bfloat16 (ties to even), as a checkpoint stores them."""
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return np.asarray(u.astype(np.uint32).view(np.float32))


def random_weights(cfg, seed=0, gain=1.0):
    """Random tensors for any configuration, already rounded to bfloat16."""
    rng = np.random.default_rng(seed)
    W, V = int(cfg["width"]), int(cfg["vocab"])

    def lin(o, i, g=1.0):
        return bf16_round(rng.standard_normal((o, i)) * (g * gain / math.sqrt(i)))

    w = {"embed": bf16_round(rng.standard_normal((V, W))), "head": lin(V, W, 2.0), "final.norm": bf16_round(rng.uniform(0.8, 1.2, ()))}
    bg = cfg.get("embedding", {}).get("bigram")
    if bg:
        w["bigram"] = bf16_round(rng.standard_normal((int(bg["buckets"]) + 1, W)) * 0.5)
    loop = cfg.get("loop")
    if loop:
        w["loop.step"] = bf16_round(rng.standard_normal((int(loop["times"]), W)) * 0.3)
    for i, layer in enumerate(cfg["layers"]):
        p, mix = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = bf16_round(rng.uniform(0.8, 1.2, ()))
        H, dk, dv = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
        if layer["type"] == "latent_attention":
            r = int(mix["kv_rank"])
            w[p + "mix.q"], w[p + "mix.dkv"] = lin(H * dk, W, 2.0), lin(r, W)
            w[p + "mix.dkv.norm"] = bf16_round(rng.uniform(0.7, 1.3, r))
            w[p + "mix.uk"], w[p + "mix.uv"] = lin(H * dk, r, 2.0), lin(H * dv, r)
            w[p + "mix.sink"] = bf16_round(rng.standard_normal(H))
            w[p + "mix.g"], w[p + "mix.o"] = lin(H, W), lin(W, H * dv)
        else:
            w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"] = lin(H * dk, W), lin(H * dk, W, 2.0), lin(H * dv, W)
            w[p + "mix.f.b"] = bf16_round(rng.standard_normal(H * dk))
            w[p + "mix.lower"] = bf16_round(rng.uniform(0.0, 0.9, H * dk))
            w[p + "mix.norm"] = bf16_round(rng.uniform(0.7, 1.3, dv))
            w[p + "mix.o"] = lin(W, H * dv)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        w[p + "norm2"] = bf16_round(rng.uniform(0.8, 1.2, ()))
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            w[p + "mlp.up"], w[p + "mlp.up.b"] = lin(ff, W), bf16_round(rng.standard_normal(ff) * 0.1)
            w[p + "mlp.down"], w[p + "mlp.down.b"] = lin(W, ff), bf16_round(rng.standard_normal(W) * 0.1)
            w[p + "mlp.act"] = bf16_round(np.array([0.6, 0.3, 0.2, 0.05]) + rng.standard_normal(4) * 0.05)
        else:
            ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            for e in range(E):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
            w[p + "mlp.router"] = lin(E, W, 3.0)
            if mlp.get("shared"):
                sf = int(mlp["shared"]["ff"])
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = lin(sf, W), lin(sf, W), lin(W, sf)
    return w
