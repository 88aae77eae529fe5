"""Plain, slow implementation of the Movarax decoder, for comparison only.

Whole sequences, no cache, one function for each mechanism, numpy only. It shares no code with the package under
test (its own file reader, its own rotation angles). Notation:

  T tokens, d width, H heads.
  norm(x; w)   = x / sqrt(mean(x^2) + eps) * w
  layer:       x += mixer(norm(x; w1));  x += ff(norm(x; w2))           (ff may be absent)
  latent attention:  q = Wq h, per head [n plain | r rotated];  z = Wd h;  c = norm(z[:R]; wn);  s = rotate(z[R:])
               key_h(j) = [Uk_h c_j | s_j],  value_h(j) = Uv_h c_j,  score = scale * q_h(i) . key_h(j),  j <= i
               p_j = exp(score_j - M) / (exp(sink_h - M) + sum_j exp(score_j - M)),   out = Wo [sum_j p_j value_h(j)]_h
               rotation: the pair (x[2i], x[2i+1]) at position t turns by the angle t * base^(-2i / dims), i < dims / 2
               A layer that names another one (kv_from) has no Wd and uses that layer's c and s.
  decay attention:  q, k, v = silu(W. h);  S <- a_h S + k v^T;  o = S^T q;  out = Wo (norm([o_h]_h; wn) * sigmoid(Wg h))
  experts:     z = R h;  s = sigmoid(z);  the `top` largest s chosen;  out = sum_e E_e(s_e h) + Shared(h),
               E(x) = Wdown relu(Wup x)^2

`rnd` (optional) is applied where a bfloat16 engine stores a tensor; with rnd=None all is `real` (float32 by
default, float64 to measure float32's own noise). latent_rows (a boolean per token, or None) marks the tokens whose
latent attention the engine takes over its cache rows (every step but a prompt from its first token): there the query
is carried into the latent space, q~_h = Uk_h^T q_h, the scores are q~_h . c_j + q_rot . s_j, and Uv_h is applied to
sum_j p_j c_j. Both forms are the same numbers; they round at different places.
"""
import json
import struct

import numpy as np


def read_safetensors(path):
    """name -> float32 array (bfloat16 widened exactly) or int32 array."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[8 + n + a:8 + n + b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").copy()
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"])
    return out


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def _keep(rnd, a):
    return a if rnd is None else rnd(a).astype(a.dtype)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ----------------------------------------------------------------- mechanisms, one function each

def norm(x, w, eps):
    r = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + x.dtype.type(eps))
    return x * r * w


def rotate_pairs(x, positions, base, dims):
    """x [..., T, n]: the pairs (2i, 2i+1), i < dims / 2, turn by positions * base^(-2i / dims); the rest stays.
    Angles are made in float64 whatever x's type."""
    out = x.copy()
    if not dims:
        return out
    i = np.arange(dims // 2, dtype=np.float64)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * np.power(float(base), -2.0 * i / dims)[None, :]
    cos, sin = np.cos(angle).astype(x.dtype), np.sin(angle).astype(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_with_sink(z, sink):
    """z [T, T] causal scores (row i sees j <= i); the sink is one more term of the denominator."""
    T = z.shape[0]
    z = np.where(np.tril(np.ones((T, T), dtype=bool)), z, -np.inf)
    top = np.maximum(z.max(axis=-1), sink)
    e = np.exp(z - top[:, None])
    return e / (e.sum(axis=-1) + np.exp(sink - top))[:, None]


def latents(h, p, m, eps, positions, rnd=None):
    """(c [T, R], s [T, r]) of a layer with a down-projection of its own."""
    R = m["kv_rank"]
    z = _keep(rnd, h @ p["dkv"].T)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    return _keep(rnd, norm(z[:, :R], p["dkv.norm"], eps)), _keep(rnd, rotate_pairs(z[:, R:], positions, rot["base"], rot["dims"]))


def latent_attention(h, p, m, c, s, positions, rnd=None, latent_rows=None):
    T, H, n, r, V = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = _keep(rnd, h @ p["q"].T).reshape(T, H, n + r)
    q_plain = q[..., :n]
    q_rot = _keep(rnd, rotate_pairs(q[..., n:].transpose(1, 0, 2), positions, rot["base"], rot["dims"]).transpose(1, 0, 2))
    uk, uv = p["uk"].reshape(H, n, -1), p["uv"].reshape(H, V, -1)
    keys = _keep(rnd, c @ p["uk"].T).reshape(T, H, n)
    values = _keep(rnd, c @ p["uv"].T).reshape(T, H, V)
    out = np.zeros((T, H, V), dtype=h.dtype)
    scale = h.dtype.type(m["scale"])
    for a in range(H):
        w = softmax_with_sink((q_plain[:, a] @ keys[:, a].T + q_rot[:, a] @ s.T) * scale, p["sink"][a])
        out[:, a] = _keep(rnd, w @ values[:, a])
        if latent_rows is not None and np.any(latent_rows):
            q_lat = _keep(rnd, q_plain[:, a] @ uk[a])
            w = softmax_with_sink((q_lat @ c.T + q_rot[:, a] @ s.T) * scale, p["sink"][a])
            out[latent_rows, a] = _keep(rnd, _keep(rnd, w @ c) @ uv[a].T)[latent_rows]
    return out.reshape(T, H * V) @ p["o"].T


def decay_recurrence(q, k, v, decay):
    """q, k [T, n], v [T, V] of one head -> o [T, V]: S <- decay S + k v^T, o = S^T q, token by token."""
    S = np.zeros((k.shape[1], v.shape[1]), dtype=q.dtype)
    o = np.zeros_like(v)
    a = q.dtype.type(decay)
    for t in range(q.shape[0]):
        S = a * S + np.outer(k[t], v[t])
        o[t] = S.T @ q[t]
    return o


def decay_attention(h, p, m, eps, real, rnd=None):
    T, H, n, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    lin = lambda name: _keep(rnd, h @ p[name].T)
    hi = lambda a: a.astype(real if rnd is None else np.float32)  # the recurrence is float32 in a bfloat16 engine
    q, k, v = hi(silu(lin("q"))).reshape(T, H, n), hi(silu(lin("k"))).reshape(T, H, n), hi(silu(lin("v"))).reshape(T, H, V)
    o = np.stack([decay_recurrence(q[:, a], k[:, a], v[:, a], m["decay"][a]) for a in range(H)], axis=1).reshape(T, H * V)
    return _keep(rnd, norm(o, p["norm"], eps) * sigmoid(lin("g"))) @ p["o"].T


def gated_feed_forward(h, p, rnd=None):
    gate, up = _keep(rnd, h @ p["gate"].T), _keep(rnd, h @ p["up"].T)
    return _keep(rnd, silu(gate) * up) @ p["down"].T


def relu_squared(z):
    return np.maximum(z, 0) ** 2


def expert(x, up, down, rnd=None, stored_before=False):
    """stored_before: the engine stores the first product before the activation too (the shared expert's runs as a
    product of its own)."""
    z = x @ up.T
    return _keep(rnd, relu_squared(_keep(rnd, z) if stored_before else z)) @ down.T


def route(h, router, top):
    """(chosen experts [T, top], their scores [T, top]): the largest sigmoid(R h), a tie to the lower index."""
    s = sigmoid(h.astype(np.float32) @ router.T.astype(np.float32))
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def routed_feed_forward(h, p, mlp, rnd=None):
    chosen, scores = route(h, p["router"], mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], scores[t]):
            out[t] += expert(_keep(rnd, h.dtype.type(s) * h[t:t + 1]), p[f"e{e}.up"], p[f"e{e}.down"], rnd)[0]
    if mlp.get("shared"):
        # (a shared expert of the routed experts' size runs with them; one of another size as products of its own)
        out += expert(h, p["shared.up"], p["shared.down"], rnd, stored_before=mlp["shared"]["ff"] != mlp["expert"]["ff"])
    return out


# ----------------------------------------------------------------- the model

def forward(config, tensors, tokens, real=np.float32, rnd=None, layers_out=None, latent_rows=None):
    """Logits [T, vocab] of a whole sequence. layers_out: a list that gets the stream after every layer."""
    W = {k: (v.astype(real) if v.dtype.kind == "f" else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = np.arange(T)
    x = W["embed"][np.asarray(tokens, dtype=np.int64)] * real((config.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    for i, layer in enumerate(config["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        p = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        hn = _keep(rnd, norm(x, W[pre + "norm1"], eps))
        if layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latents(hn, p, m, eps, positions, rnd)
            c, s = kept[m["kv_from"] if m.get("kv_from") is not None else i]
            rows = latent_rows.get(i) if isinstance(latent_rows, dict) else latent_rows   # (may differ by layer)
            x = x + latent_attention(hn, p, m, c, s, positions, rnd, rows)
        else:
            x = x + decay_attention(hn, p, m, eps, real, rnd).astype(real)
        if layer.get("mlp") is not None:
            p = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            hn = _keep(rnd, norm(x, W[pre + "norm2"], eps))
            x = x + (gated_feed_forward(hn, p, rnd) if layer["mlp"].get("kind", "dense") == "dense"
                     else routed_feed_forward(hn, p, layer["mlp"], rnd))
        if layers_out is not None:
            layers_out.append(x.copy())
    return _keep(rnd, norm(x, W["final.norm"], eps)) @ W["head"].T


def generate(config, tensors, prompt, n_new):
    """Greedy continuation, the whole sequence recomputed for every token."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]
