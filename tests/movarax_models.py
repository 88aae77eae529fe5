"""Small Movarax models for the tests: configurations that differ in every size and option, and random weights made
here (numpy, bfloat16-representable), written as a model folder."""
import json
import os

import numpy as np
import torch

from plain import movarax_plain as plain


def latent_layer(heads, dim, rot_dim, vdim, rank, scale, rot=None, kv_from=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot:
        mixer["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def decay_layer(kind, heads, dim, vdim, decay, mlp=None):
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(n, top, ff, shared=None):
    mlp = {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


# U: a recurrent layer first (three heads, values smaller than keys) with two of five experts and a shared one; latent
#    attention whose bfloat16 prompts run in full size (heads of 24 + 8, values of 16, 40 latents), dense feed-forward;
#    a layer that reads layer 1's latents with other heads (four of 8 + 8) and no feed-forward at all; a recurrent layer
#    under its second name, one head of 40 channels (two registers a thread), all three experts chosen, none shared.
# V: sizes that fit no vector: heads of 10 + 6 of which 4 dimensions rotate, values of 7, 21 latents (a cache row padded
#    to 32), one of four experts; a recurrent layer with 5 channels, values of 3 and a head that never forgets; a layer
#    reading layer 0's latents with a single head whose values are larger than its keys.
# W: every latent layer with latents of its own, two of them the same sizes (one cache group, two entries); one expert
#    of one (the router chooses nothing but still weighs); heads of 4 + 16, mostly rotated, that no vector kernel takes.
CONFIGS = {
    "U": {"architecture": "Movarax", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
          "layers": [decay_layer("lightning", 3, 16, 8, (0.9, 0.5, 0.99), experts(5, 2, 24, 40)),
                     latent_layer(2, 24, 8, 16, 40, 0.35, rot=(10000.0, 8), mlp=dense(96)),
                     latent_layer(4, 8, 8, 8, 40, 0.5, rot=(10000.0, 8), kv_from=1),
                     decay_layer("lightning_2", 1, 40, 24, (0.97,), experts(3, 3, 16))]},
    "V": {"architecture": "Movarax", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
          "layers": [latent_layer(3, 10, 6, 7, 21, 0.4, rot=(100.0, 4), mlp=experts(4, 1, 12, 9)),
                     decay_layer("lightning", 2, 5, 3, (0.8, 1.0), dense(20)),
                     latent_layer(1, 12, 6, 20, 21, 0.3, rot=(100.0, 4), kv_from=0, mlp=experts(2, 2, 8, 8))]},
    "W": {"architecture": "Movarax", "vocab": 77, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.25},
          "layers": [latent_layer(2, 8, 8, 8, 16, 0.4, rot=(250000.0, 8), mlp=experts(1, 1, 8)),
                     latent_layer(2, 8, 8, 8, 16, 0.4, rot=(250000.0, 8), mlp=dense(40)),
                     latent_layer(2, 4, 16, 8, 24, 0.3, rot=(50.0, 16))]},
}


def random_config(rng):
    """A random configuration: two to five layers of either mixer, heads of 1 to 32, sizes that fit and that do not fit
    the vector kernels, rotations of part or none of the rotated part, layers that read an earlier layer's latents, every
    kind of feed-forward or none."""
    width = int(rng.choice([24, 32, 40, 64, 72, 96, 128]))
    n_layers = int(rng.integers(2, 6))
    layers, latent_at = [], []
    for i in range(n_layers):
        kind = rng.choice(['latent', 'decay'])
        r = rng.random()
        if r < 0.25: mlp = None
        elif r < 0.5: mlp = dense(int(rng.choice([16, 24, 40, 64])))
        else:
            E = int(rng.choice([1, 2, 3, 4, 8, 16])); top = int(rng.integers(1, min(E, 4) + 1)); ff = int(rng.choice([8, 12, 16, 24, 32]))
            shared = None if rng.random() < 0.3 else (ff if rng.random() < 0.6 else int(rng.choice([8, 16, 20])))
            mlp = experts(E, top, ff, shared)
        if kind == 'latent':
            own = [j for j in latent_at if 'kv_from' not in layers[j]['mixer']]
            if own and rng.random() < 0.4:
                j = int(rng.choice(own)); src = layers[j]['mixer']
                H = int(rng.choice([1, 2, 3, 4, 8, 17, 24])); dim = int(rng.choice([1, 4, 8, 12, 16, 32])); vdim = int(rng.choice([3, 8, 16, 24, 40]))
                rot = (src['rot']['base'], src['rot']['dims']) if 'rot' in src else None
                layers.append(latent_layer(H, dim, src['rot_dim'], vdim, src['kv_rank'], 0.3, rot=rot, kv_from=j, mlp=mlp))
            else:
                H = int(rng.choice([1, 2, 3, 4, 8, 17, 24, 32])); dim = int(rng.choice([1, 4, 8, 12, 16, 32, 64]))
                rot_dim = int(rng.choice([0, 2, 4, 8, 16, 32])); vdim = int(rng.choice([3, 8, 16, 24, 40, 136]))
                rank = int(rng.choice([5, 8, 16, 24, 32, 48, 96, 160]))
                dims = int(rng.choice([d for d in (0, 2, 4, 8, 16, 32) if d <= rot_dim]))
                rot = (float(rng.choice([100.0, 10000.0, 1e6])), dims) if dims else None
                layers.append(latent_layer(H, dim, rot_dim, vdim, rank, float(rng.choice([0.2, 0.35, 0.5])), rot=rot, mlp=mlp))
            latent_at.append(i)
        else:
            H = int(rng.choice([1, 2, 3, 5, 8])); dim = int(rng.choice([1, 5, 16, 24, 64, 100, 128, 130])); vdim = int(rng.choice([1, 3, 8, 20, 32, 130]))
            decay = [float(x) for x in rng.choice([0.0, 0.3, 0.9, 0.99, 0.999, 1.0], H)]
            layers.append(decay_layer(str(rng.choice(['lightning', 'lightning_2'])), H, dim, vdim, decay, mlp))
    return {"architecture": "Movarax", "vocab": int(rng.choice([50, 131, 300])), "width": width, "norm": {"eps": float(rng.choice([1e-6, 1e-5]))},
            "embedding": {"scale": float(rng.choice([0.5, 1.0, 3.0]))}, "layers": layers}


def config(name):
    return json.loads(json.dumps(CONFIGS[name]))


def _bf16(a):
    return plain.bf16_round(np.asarray(a, dtype=np.float32))


def weights(name, seed=0):
    """{tensor name: float32 array of bfloat16-representable values}. Matrices are scaled by their input size so that
    activations stay of order one; queries and latents are made large so that scores are a few units wide and a lost
    or extra key shows."""
    raw = config(name)
    rng = np.random.default_rng(seed)
    d = raw["width"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)
    w["embed"] = rng.standard_normal((raw["vocab"], d))
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = 1.0 + rng.standard_normal(d) * 0.1
        if layer["type"] == "latent_attention":
            H, n, r, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = mat(H * (n + r), d, 2.0)
            if "kv_from" not in m:
                w[p + "mix.dkv"] = mat(R + r, d, 2.0)
                w[p + "mix.dkv.norm"] = 1.5 + rng.standard_normal(R) * 0.2
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * n, R, 1.5), mat(H * V, R, 2.0)
            w[p + "mix.sink"] = rng.standard_normal(H)
            w[p + "mix.o"] = mat(d, H * V, 2.0)
        else:
            H, n, V = m["heads"], m["dim"], m["vdim"]
            for t, rows in (("q", H * n), ("k", H * n), ("v", H * V), ("g", H * V)):
                w[p + "mix." + t] = mat(rows, d, 2.0)
            w[p + "mix.norm"] = 1.0 + rng.standard_normal(H * V) * 0.1
            w[p + "mix.o"] = mat(d, H * V, 2.0)
        mlp = layer["mlp"]
        if mlp is not None:
            w[p + "norm2"] = 1.0 + rng.standard_normal(d) * 0.1
            if mlp["kind"] == "dense":
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(mlp["ff"], d), mat(mlp["ff"], d), mat(d, mlp["ff"], 2.0)
            else:
                w[p + "mlp.router"] = mat(mlp["router"]["experts"], d, 3.0)
                for e in range(mlp["router"]["experts"]):
                    w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = mat(mlp["expert"]["ff"], d, 1.5), mat(d, mlp["expert"]["ff"], 1.5)
                if mlp.get("shared"):
                    w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(mlp["shared"]["ff"], d), mat(d, mlp["shared"]["ff"])
    w["final.norm"] = 1.0 + rng.standard_normal(d) * 0.1
    w["head"] = mat(raw["vocab"], d, 2.0)
    return {n: _bf16(t) for n, t in w.items()}


def write_folder(tmp, name, seed=0, tensors=None):
    """config.json and model.safetensors of configuration `name` under tmp -> (folder, config dict, tensors)."""
    from abacus_b200.weights.safetensors_io import save_tensors
    raw = config(name)
    tensors = tensors if tensors is not None else weights(name, seed)
    folder = os.path.join(str(tmp), f"movarax{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {n: torch.from_numpy(np.ascontiguousarray(t)).to(torch.bfloat16) for n, t in tensors.items()})
    return folder, raw, tensors
