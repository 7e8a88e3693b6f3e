"""Katadra on the B200 engine: a decoder-only language model whose configuration lists its layers.

A checkpoint directory holds `config.json` (`architecture: "Katadra"`, `width`, `vocab`, `norm.eps`, `layers`) and
`model.safetensors`. Each entry of `layers` names its mixer (`mamba2`, or `parallel` = attention + RWKV time mixing side by
side), the mixer's sizes, its feed-forward (`mlp`, or null) and optionally `weights_of: j` (the layer computes with layer
j's tensors on a state of its own). This module only reads the configuration; tensors, engine, generation and replay are the
layer-list decoders' common code (layer_list.py).
"""
from ..._b2 import MIXER_MAMBA2, MIXER_PARALLEL
from .layer_list import LayerListConfig, LayerListForCausalLM, TraceSession, read_safetensors  # noqa: F401 (re-exported)


class KatadraConfig(LayerListConfig):
    model_type = "Katadra"

    def owner(self, i):
        """The layer whose tensors layer i computes with (itself, unless `weights_of` names another; chains are followed)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None and int(self.layers[i]["weights_of"]) != i:
            if i in seen:
                raise ValueError(f"weights_of of layer {i} never reaches a layer that owns its tensors")
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
        return i

    def layer_descs(self, shapes):
        """Engine descriptions of the layers. Sizes the configuration does not spell out (rows of the distance-bias table, rank
        of the decay projection) are read from the tensor shapes."""
        out = []
        for i, layer in enumerate(self.layers):
            src, mix, mlp = self.owner(i), layer["mixer"], layer.get("mlp")
            d = dict(weights_of=-1 if src == i else src, ff=0)
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
                d["ff"] = int(mlp["ff"])
            if layer["type"] == "mamba2":
                d.update(type=MIXER_MAMBA2, m_heads=int(mix["heads"]), m_vdim=int(mix["vdim"]), m_state=int(mix["state"]),
                         m_groups=int(mix["groups"]), m_conv=int(mix["conv"]), m_norm_groups=int(mix["norm_groups"]))
            elif layer["type"] == "parallel":
                a, r = mix["left"], mix["right"]
                rel, w1 = shapes.get(f"l{src}.mix.left.rel"), shapes.get(f"l{src}.mix.right.w1")
                if rel is None or w1 is None:
                    raise ValueError(f"layer {i}: the checkpoint has no l{src}.mix.left.rel / l{src}.mix.right.w1")
                d.update(type=MIXER_PARALLEL, a_heads=int(a["heads"]), a_kv_heads=int(a["kv_heads"]), a_dim=int(a["dim"]),
                         a_vdim=int(a["vdim"]), a_rel_rows=int(rel[0]), a_bias_max=float(a["bias_max"]), a_scale=float(a["scale"]),
                         a_softcap=float(a["softcap"]), a_temp_coef=float(a["q_temp"]["coef"]), a_temp_every=float(a["q_temp"]["every"]),
                         r_heads=int(r["heads"]), r_dim=int(r["dim"]), r_decay_rank=int(w1[0]),
                         left_scale=float(mix["left_scale"]), right_scale=float(mix["right_scale"]))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {layer['type']!r}")
            out.append(d)
        return out


class KatadraForCausalLM(LayerListForCausalLM):
    """Holds the checkpoint tensors (CPU) and builds the device engine on first use.

    dtype: torch.bfloat16 = bf16 matrix products with fp32 accumulation on bf16 weights (norms, scores, recurrences, the
    residual stream in fp32); torch.float32 = everything in true fp32."""
    config_class = KatadraConfig
