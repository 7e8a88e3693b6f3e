"""Pefivik on the B200 engine: a pre-norm layer-list decoder with a hashed bigram embedding and a looped block of layers.

`config.json`: `architecture: "Pefivik"`, `width`, `vocab`, `norm.eps`, `residual_mult`, `logit_softcap`,
`embedding.bigram {buckets, mul_prev, mul_cur}`, `loop {start, stop, times}` and `layers`. A layer is
`x += m * mixer(g1 * unit_rms(x))`, then `x += m * ff(g2 * unit_rms(x))` with ONE learned number per norm. Mixers:
`latent_attention` (no positions; keys and values are read off one cached low-rank row per token; a per-head sink in the
softmax denominator; a per-head sigmoid output gate) and `hgrn2` (a gated linear recurrence whose forget gate, bounded below,
also decides what is written). Feed-forwards: `dense` (biased projections around PolyNorm) and `moe` (sigmoid router,
group-limited top-k, SiLU-gated experts, a shared expert). Layers `start .. stop-1` run `times` times with the same tensors,
every pass on a cache/state of its own; from the second pass on the embedding output is added again, and a learned vector
`loop.step[t]` before every pass. The logits are soft-capped with tanh. This module only reads the configuration; tensors,
engine, generation and replay are the layer-list decoders' common code (layer_list.py).
"""
from ..._b2 import BLOCK_PRE_RMS1, FF_MOE, FF_POLYNORM, MIXER_HGRN2, MIXER_LATENT_ATTN
from .layer_list import LayerListConfig, LayerListForCausalLM


class PefivikConfig(LayerListConfig):
    model_type = "Pefivik"

    def model_desc(self):
        c = self.raw
        d = dict(block=BLOCK_PRE_RMS1, residual_mult=float(c.get("residual_mult", 1.0)), logit_softcap=float(c.get("logit_softcap") or 0.0))
        bg = (c.get("embedding") or {}).get("bigram")
        if bg:
            d.update(bigram_buckets=int(bg["buckets"]), bigram_mul_prev=int(bg["mul_prev"]), bigram_mul_cur=int(bg["mul_cur"]))
        loop = c.get("loop")
        if loop and int(loop["stop"]) > int(loop["start"]):
            if int(loop["times"]) < 1:
                raise ValueError("loop.times must be at least 1")
            d.update(loop_start=int(loop["start"]), loop_stop=int(loop["stop"]), loop_times=int(loop["times"]))
        return d

    def layer_descs(self, shapes):
        out = []
        for i, layer in enumerate(self.layers):
            mix, mlp = layer["mixer"], layer.get("mlp")
            d = dict(weights_of=-1, ff=0)
            if layer["type"] == "latent_attention":
                d.update(type=MIXER_LATENT_ATTN, la_heads=int(mix["heads"]), la_dim=int(mix["dim"]), la_vdim=int(mix["vdim"]),
                         la_rank=int(mix["kv_rank"]), la_scale=float(mix["scale"]))
            elif layer["type"] == "hgrn2":
                d.update(type=MIXER_HGRN2, g_heads=int(mix["heads"]), g_dim=int(mix["dim"]), g_vdim=int(mix["vdim"]))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {layer['type']!r}")
            if mlp:
                kind = mlp.get("kind", "dense")
                if kind == "dense":
                    d.update(ff_kind=FF_POLYNORM, ff=int(mlp["ff"]))
                elif kind == "moe":
                    r = mlp["router"]
                    groups = r.get("groups") or {"count": 1, "keep": 1}
                    d.update(ff_kind=FF_MOE, ff=int(mlp["expert"]["ff"]), moe_experts=int(r["experts"]), moe_top=int(r["top"]),
                             moe_groups=int(groups["count"]), moe_keep=int(groups["keep"]), moe_scale=float(r.get("scale", 1.0)),
                             moe_shared_ff=int(mlp["shared"]["ff"]) if mlp.get("shared") else 0)
                else:
                    raise NotImplementedError(f"layer {i}: feed-forward kind {kind!r}")
            out.append(d)
        return out


class PefivikForCausalLM(LayerListForCausalLM):
    """Holds the checkpoint tensors (CPU) and builds the device engine on first use.

    dtype: torch.bfloat16 = bf16 matrix products with fp32 accumulation on bf16 weights (norms, router, scores and softmax, the
    latent cache, gates and state of the recurrence, the residual stream in fp32); torch.float32 = everything in true fp32."""
    config_class = PefivikConfig
