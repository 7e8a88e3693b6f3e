"""Plain, slow restatement of the Katadra decoder in PyTorch on the CPU: one function per mechanism, token-by-token loops
where the design has a recurrence, no caches shared with the product path. Test infrastructure only.

Katadra is a decoder-only language model whose layers come from a list in its configuration. Every layer applies its
normalisation to the OUTPUT of a sublayer (x += LayerNorm(mixer(x)); x += LayerNorm(ff(x)) when it has a feed-forward), and
a layer may borrow the weights of an earlier one while keeping a state of its own. Two mixers exist:

  mamba2    in-projection -> [z | x | B | C | dt], causal depthwise convolution + SiLU over (x, B, C), scalar-decay state-space
            recurrence per head, gate by SiLU(z), grouped RMS norm, out-projection
  parallel  the weighted sum of (left) softmax attention without rotation — unit-RMS q and k, a position-dependent query
            temperature, tanh soft-capping, a learned log-bucketed distance bias, sigmoid output gate — and (right) an
            RWKV-style token-shift + per-channel-decay linear recurrence with a current-token bonus

Everything here runs in one dtype (float64 by default) so that it can judge both number formats of the engine.
"""
import math

import torch

SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def distance_bucket(n, rows, far):
    """Row of the distance-bias table for distance n >= 0: exact up to rows // 2, logarithmic up to `far`, then the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log(math.floor((p + 1) / every) + 1)


def attention_left(h, W, c, eps):
    """h [T, width] -> [T, width]; W: dict of this mixer's tensors (q, k, v, rel, g, o)."""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms((h @ W["q"].T).view(T, H, dk), eps)
    k = unit_rms((h @ W["k"].T).view(T, G, dk), eps)
    v = (h @ W["v"].T).view(T, G, dv)
    temp = torch.tensor([query_temperature(p, c["q_temp"]["coef"], c["q_temp"]["every"]) for p in range(T)], dtype=h.dtype)
    q = q * temp[:, None, None]
    rows = W["rel"].shape[0]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, hd]) * c["scale"]
            s = c["softcap"] * torch.tanh(s / c["softcap"])
            s = s + torch.stack([W["rel"][distance_bucket(i - j, rows, c["bias_max"]), hd] for j in range(i + 1)])
            p = torch.softmax(s, 0)
            out[i, hd] = p @ v[: i + 1, g]
    gate = torch.sigmoid(h @ W["g"].T)
    return (out.reshape(T, H * dv) * gate) @ W["o"].T


def rwkv_right(h, W, c, eps):
    """Token-shift mixes, per-channel decay recurrence with a bonus for the current token, per-head unit RMS, gate."""
    T, width = h.shape
    H, d = c["heads"], c["dim"]
    prev = torch.cat([torch.zeros(1, width, dtype=h.dtype), h[:-1]], 0)
    mix = {s: h + (prev - h) * W["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W["r"].T).view(T, H, d)
    k = (mix["k"] @ W["k"].T).view(T, H, d)
    v = (mix["v"] @ W["v"].T).view(T, H, d)
    gate = silu(mix["g"] @ W["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W["w1"].T) @ W["w2"].T + W["w0"])).view(T, H, d)
    u = W["u"].view(H, d)
    S = torch.zeros(H, d, d, dtype=h.dtype)  # [head, key channel, value channel]
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    o = unit_rms(o, eps).reshape(T, H * d)
    return (o * W["norm"] * gate) @ W["o"].T


def parallel_mixer(h, W, c, eps):
    left = attention_left(h, {k[5:]: v for k, v in W.items() if k.startswith("left.")}, c["left"], eps)
    right = rwkv_right(h, {k[6:]: v for k, v in W.items() if k.startswith("right.")}, c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def mamba2_mixer(h, W, c, eps):
    T = h.shape[0]
    H, P, N, G, taps = c["heads"], c["vdim"], c["state"], c["groups"], c["conv"]
    inner = H * P
    proj = h @ W["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    pad = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], 0)
    conv = torch.stack([(pad[t:t + taps].T * W["conv"]).sum(-1) for t in range(T)]) + W["conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, P)
    Bm = conv[:, inner:inner + G * N].view(T, G, N)
    Cm = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W["dt_bias"])
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    grp = [hd // (H // G) for hd in range(H)]
    for t in range(T):
        a = torch.exp(-torch.exp(W["A_log"]) * dt[t])
        S = a[:, None, None] * S + dt[t][:, None, None] * Bm[t, grp][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Cm[t, grp]) + W["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    ng = c["norm_groups"]
    y = unit_rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def feed_forward(h, W):
    return torch.relu(h @ W["up"].T) ** 2 @ W["down"].T


def forward(cfg, weights, tokens, dtype=torch.float64, return_layers=False):
    """tokens: list of ints -> logits [T, vocab] (and the residual stream after every layer run)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    trace = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        src = i if src is None else src
        pre = f"l{src}."
        mix = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mix.")}
        m = mamba2_mixer(x, mix, layer["mixer"], eps) if layer["type"] == "mamba2" else parallel_mixer(x, mix, layer["mixer"], eps)
        x = x + layer_norm(m, w[pre + "norm1"], w[pre + "norm1.b"], eps)
        if layer.get("mlp"):
            f = feed_forward(x, {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mlp.")})
            x = x + layer_norm(f, w[pre + "norm2"], w[pre + "norm2.b"], eps)
        trace.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    return (logits, torch.stack(trace)) if return_layers else logits


def random_weights(cfg, seed=0, scale=1.0):
    """Random bf16-representable tensors with the names and shapes a checkpoint of this configuration has."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).bfloat16().float()

    w = {"embed": rnd(vocab, width), "head": rnd(vocab, width, s=width ** -0.5),
         "final.norm": 1 + rnd(width, s=0.1), "final.norm.b": rnd(width, s=0.1)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, c = f"l{i}.", layer["mixer"]
        w[p + "norm1"], w[p + "norm1.b"] = 1 + rnd(width, s=0.1), rnd(width, s=0.1)
        ws = scale * width ** -0.5
        if layer["type"] == "mamba2":
            H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            w[p + "mix.in"] = rnd(2 * inner + 2 * G * N + H, width, s=ws)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = rnd(ch, c["conv"], s=0.5), rnd(ch, s=0.1)
            w[p + "mix.dt_bias"], w[p + "mix.A_log"], w[p + "mix.D"] = rnd(H, s=0.5), rnd(H, s=0.5), rnd(H)
            w[p + "mix.norm"], w[p + "mix.o"] = 1 + rnd(inner, s=0.1), rnd(width, inner, s=inner ** -0.5)
        else:
            a, r = c["left"], c["right"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"] = rnd(a["heads"] * a["dim"], width, s=ws), rnd(a["kv_heads"] * a["dim"], width, s=ws)
            w[q + "v"], w[q + "g"] = rnd(a["kv_heads"] * a["vdim"], width, s=ws), rnd(a["heads"] * a["vdim"], width, s=ws)
            w[q + "rel"] = rnd(a.get("rel_rows", 16), a["heads"])
            w[q + "o"] = rnd(width, a["heads"] * a["vdim"], s=(a["heads"] * a["vdim"]) ** -0.5)
            q, n = p + "mix.right.", r["heads"] * r["dim"]
            for s_ in "rkvgw":
                w[q + "mu." + s_] = torch.rand(width, generator=g).bfloat16().float()
            for s_ in "rkvg":
                w[q + s_] = rnd(n, width, s=ws)
            rank = r.get("decay_rank", 8)
            w[q + "w1"], w[q + "w2"], w[q + "w0"] = rnd(rank, width, s=ws), rnd(n, rank, s=rank ** -0.5), rnd(n, s=0.5) - 1.0
            w[q + "u"], w[q + "norm"], w[q + "o"] = rnd(r["heads"], r["dim"], s=0.5), 1 + rnd(n, s=0.1), rnd(width, n, s=n ** -0.5)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            w[p + "norm2"], w[p + "norm2.b"] = 1 + rnd(width, s=0.1), rnd(width, s=0.1)
            w[p + "mlp.up"], w[p + "mlp.down"] = rnd(ff, width, s=ws), rnd(width, ff, s=ff ** -0.5)
    return {k: v.bfloat16().float() for k, v in w.items()}
