"""Host side of the Katadra path (no GPU): configuration reader, model registry, checkpoint reader, oracle sanity."""
import json
import math
import os
import struct
import subprocess
import sys

import pytest
import torch

from oracle import katadra_oracle as O

CFG = {"architecture": "Katadra", "width": 24, "vocab": 40, "norm": {"eps": 1e-5}, "layers": [
    {"type": "mamba2", "mixer": {"heads": 2, "vdim": 6, "state": 5, "groups": 1, "conv": 3, "norm_groups": 2}, "mlp": None},
    {"type": "parallel", "mlp": {"kind": "dense", "ff": 30},
     "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 5, "vdim": 3, "bias_max": 20, "scale": 0.4, "softcap": 5.0,
                        "q_temp": {"coef": 0.5, "every": 3}, "rel_rows": 6},
               "right": {"heads": 2, "dim": 6, "decay_rank": 4}, "left_scale": 0.5, "right_scale": 2.0}},
    {"type": "mamba2", "mixer": {"heads": 2, "vdim": 6, "state": 5, "groups": 1, "conv": 3, "norm_groups": 2}, "mlp": None,
     "weights_of": 0}]}


def write_checkpoint(path, cfg, weights):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for k, v in weights.items():
        raw = v.bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def test_registry_config_reader_and_checkpoint_reader(tmp_path):
    from llava.model import MODEL_REGISTRY, KatadraConfig, model_class_for
    from llava.model.language_model.katadra import read_safetensors
    from llava._b2 import MIXER_MAMBA2, MIXER_PARALLEL

    w = O.random_weights(CFG, seed=3)
    write_checkpoint(str(tmp_path), CFG, w)
    assert "Katadra" in MODEL_REGISTRY and model_class_for(str(tmp_path)).__name__ == "KatadraForCausalLM"
    sd = read_safetensors(os.path.join(str(tmp_path), "model.safetensors"))
    assert set(sd) == set(w) and all(torch.equal(sd[k].float(), w[k]) for k in w)
    assert not any(k.startswith("l2.") for k in sd), "a layer that borrows weights has no tensors"
    c = KatadraConfig.from_pretrained(str(tmp_path))
    descs = c.layer_descs({k: tuple(v.shape) for k, v in sd.items()})
    assert [d["type"] for d in descs] == [MIXER_MAMBA2, MIXER_PARALLEL, MIXER_MAMBA2]
    assert [d["weights_of"] for d in descs] == [-1, -1, 0] and [d["ff"] for d in descs] == [0, 30, 0]
    assert descs[1]["a_rel_rows"] == 6 and descs[1]["r_decay_rank"] == 4 and descs[1]["a_temp_every"] == 3.0
    with pytest.raises(ValueError):
        KatadraConfig(**dict(CFG, architecture="other"))
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump({"architecture": "nobody"}, f)
    with pytest.raises(NotImplementedError):
        model_class_for(str(tmp_path))


def test_oracle_is_causal_and_its_pieces_compose():
    """Logits of a prefix do not change when tokens follow; a layer that borrows weights computes with them on its own state."""
    w = O.random_weights(CFG, seed=4)
    toks = [3, 17, 5, 5, 29, 0, 11, 38, 2, 2, 7]
    full, layers = O.forward(CFG, w, toks, return_layers=True)
    part = O.forward(CFG, w, toks[:6])
    assert torch.allclose(full[:6], part, atol=1e-10)
    assert layers.shape == (3, len(toks), CFG["width"])
    assert not torch.allclose(layers[0], layers[2] - layers[1] + layers[0] * 0 + layers[0])  # layer 2 sees another input


def test_distance_buckets_and_query_temperature():
    rows, far = 16, 120
    b = [O.distance_bucket(n, rows, far) for n in range(400)]
    assert b[:8] == list(range(8)) and b[8] == 8 and all(x <= y for x, y in zip(b, b[1:]))
    assert b[119] == 15 and b[120] == 15 and b[399] == 15 and max(b) == 15
    assert O.distance_bucket(3, 7, 12) == 3 and O.distance_bucket(11, 7, 12) == 6
    assert O.query_temperature(0, 0.5, 256) == 1.0 and O.query_temperature(254, 0.5, 256) == 1.0
    assert math.isclose(O.query_temperature(255, 0.5, 256), 1 + 0.5 * math.log(2))
    assert math.isclose(O.query_temperature(4, 2.0, 1), 1 + 2.0 * math.log(6))


def test_trace_runner_describes_itself(repo_root):
    out = subprocess.run([sys.executable, os.path.join(repo_root, "bin", "trace_run"), "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "--max-tokens" in out.stdout and "done <step>" in out.stdout
    assert os.access(os.path.join(repo_root, "bin", "trace_run"), os.X_OK)
