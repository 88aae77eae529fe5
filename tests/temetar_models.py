"""Small Temetar models for the tests: configurations that differ in every size and option, and random weights made
here (numpy, bfloat16-representable), written as a model folder."""
import json
import os

import numpy as np
import torch

from plain import temetar_plain as plain


def attention_layer(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        mixer["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask:
        mixer["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def delta_layer(heads, kv_heads, dim, vdim, conv, ranks, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}, "_ranks": ranks}


# P: three streams, a looped middle, pairs table; attention with grouped heads, values larger than keys, part of a head
#    rotated, a window of 12 that keeps 3 first keys; a delta rule with shared key heads, 16 key channels, 4 taps.
# Q: no streams key (plain residual sum with a multiplier), no pairs table, no loop; a delta rule first, with 40 key
#    channels (two lanes to a column), values of 20, 2 taps; attention with one kv head per head, values as large as
#    keys, the whole head rotated, no window at all, then one with a window of 70 that crosses page borders.
# R: one learned stream, a loop that repeats a single layer three times, a window of 64 keeping 64 (a whole page),
#    no rotation, values of 12 (a row of q, k and v that needs padding).
CONFIGS = {
    "P": {"architecture": "Temetar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "streams": 3,
          "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 13}},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [attention_layer(4, 2, 16, 24, 0.3, rot=(10000.0, 8), mask=(12, 3), ff=96),
                     delta_layer(4, 2, 16, 8, 4, (8, 16)),
                     attention_layer(4, 2, 16, 24, 0.3, rot=(10000.0, 8), mask=(12, 3)),
                     delta_layer(4, 2, 16, 8, 4, (8, 16), ff=80)]},
    "Q": {"architecture": "Temetar", "vocab": 150, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
          "embedding": {"scale": 1.0},
          "layers": [delta_layer(3, 3, 40, 20, 2, (12, 5), ff=64),
                     attention_layer(3, 3, 32, 32, 0.2, rot=(50000.0, 32), ff=128),
                     attention_layer(6, 2, 24, 40, 0.25, rot=(777.0, 12), mask=(70, 0))]},
    "R": {"architecture": "Temetar", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "streams": 1,
          "embedding": {"scale": 2.0, "bigram": {"buckets": 31, "mul_prev": 3, "mul_cur": 5}},
          "loop": {"start": 0, "stop": 1, "times": 3},
          "layers": [attention_layer(2, 1, 32, 12, 0.18, mask=(64, 64), ff=64),
                     delta_layer(2, 1, 72, 40, 3, (4, 4))]},
    # S: sizes that fit no vector: attention heads of 20 with values of 7 (a row of 67, padded), 6 dimensions rotated,
    #    a window of 5 keeping 1; a delta rule with 5 key channels, values of 3, 5 taps; two streams.
    "S": {"architecture": "Temetar", "vocab": 61, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 1.3, "streams": 2,
          "embedding": {"scale": 0.5, "bigram": {"buckets": 7, "mul_prev": 1000003, "mul_cur": 999983}},
          "layers": [attention_layer(2, 1, 20, 7, 0.2, rot=(100.0, 6), mask=(5, 1), ff=24),
                     delta_layer(2, 1, 5, 3, 5, (3, 2))]},
}


def config(name):
    """(config.json's dict, {layer index: (decay rank, gate rank)})."""
    raw = json.loads(json.dumps(CONFIGS[name]))
    ranks = {i: tuple(layer.pop("_ranks")) for i, layer in enumerate(raw["layers"]) if "_ranks" in layer}
    return raw, ranks


def _bf16(a):
    return plain.bf16_round(np.asarray(a, dtype=np.float32))


def weights(name, seed=0):
    """{tensor name: float32 array of bfloat16-representable values}. Matrices are scaled by their input size so that
    activations stay of order one; q/k norm weights are large so that scores are a few units wide and a lost or
    extra key shows."""
    raw, ranks = config(name)
    rng = np.random.default_rng(seed)
    d, s = raw["width"], raw.get("streams")
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)
    w["embed"] = rng.standard_normal((raw["vocab"], d))
    big = raw["embedding"].get("bigram")
    if big:
        w["bigram"] = rng.standard_normal((big["buckets"] + 1, d)) * raw["embedding"]["scale"] * 0.5
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = rng.standard_normal(d) * 0.1
        if layer["type"] == "attention":
            w[p + "mix.q"] = mat(m["heads"] * m["dim"], d)
            w[p + "mix.k"] = mat(m["kv_heads"] * m["dim"], d)
            w[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], d, 2.0)
            w[p + "mix.q.norm"] = 2.0 + rng.standard_normal(m["dim"]) * 0.2
            w[p + "mix.k.norm"] = 2.0 + rng.standard_normal(m["dim"]) * 0.2
            w[p + "mix.sink"] = rng.standard_normal(m["heads"])
            w[p + "mix.o"] = mat(d, m["heads"] * m["vdim"], 2.0)
        else:
            ra, rg = ranks[i]
            gk, hv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(gk, d, 2.0), mat(gk, d, 2.0), mat(hv, d, 2.0)
            for n, c in (("q", gk), ("k", gk), ("v", hv)):
                w[p + f"mix.{n}.conv"] = 0.4 + rng.standard_normal((c, m["conv"])) * 0.4
            w[p + "mix.b"] = mat(m["heads"], d, 2.0)
            w[p + "mix.A_log"] = rng.standard_normal(m["heads"]) * 0.5 - 1.0
            w[p + "mix.norm"] = 1.0 + rng.standard_normal(m["vdim"]) * 0.1
            w[p + "mix.a1"], w[p + "mix.a2"] = mat(ra, d), mat(m["heads"] * m["dim"], ra, 2.0)
            w[p + "mix.dt_bias"] = rng.standard_normal(m["heads"] * m["dim"]) * 0.5
            w[p + "mix.g1"], w[p + "mix.g2"] = mat(rg, d), mat(hv, rg, 2.0)
            w[p + "mix.o"] = mat(d, hv, 2.0)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = rng.standard_normal(d) * 0.1
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, d), mat(ff, d), mat(d, ff, 2.0)
        if s:
            for q in (1, 2) if layer["mlp"] is not None else (1,):
                w[p + f"hc{q}.in"] = 1.0 / s + rng.standard_normal(s) * 0.2 / s
                w[p + f"hc{q}.out"] = 1.0 + rng.standard_normal(s) * 0.2
                w[p + f"hc{q}.mix"] = np.eye(s) + rng.standard_normal((s, s)) * 0.1
    w["final.norm"] = rng.standard_normal(d) * 0.1
    w["head"] = mat(raw["vocab"], d, 2.0)
    return {n: _bf16(t) for n, t in w.items()}


def write_folder(tmp, name, seed=0, tensors=None):
    """config.json and model.safetensors of configuration `name` under tmp -> (folder, config dict, tensors)."""
    from abacus_b200.weights.safetensors_io import save_tensors
    raw, _ = config(name)
    tensors = tensors if tensors is not None else weights(name, seed)
    folder = os.path.join(str(tmp), f"temetar{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {n: torch.from_numpy(np.ascontiguousarray(t)).to(torch.bfloat16) for n, t in tensors.items()})
    return folder, raw, tensors
