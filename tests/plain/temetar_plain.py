"""Plain, slow implementation of the Temetar decoder, for comparison only.

Whole sequences, no cache, one function for each mechanism, numpy only. It shares no code with the
package under test (its own file reader, its own rotation angles). Notation used below:

  T tokens, d width, s residual streams, m the branch multiplier.
  norm1p(x; w)  = x / sqrt(mean(x^2) + eps) * (1 + w)            (layer norms and the last norm)
  norm(x; w)    = x / sqrt(mean(x^2) + eps) * w                  (per-head norms inside the mixers)
  streams:  u = sum_s a[s] X[s];  y = branch(norm1p(u));  X'[t] = sum_s M[s, t] X[s] + m c[t] y
  delta:    S <- diag(g) S;  e = b (v - S^T k);  S <- S + k e^T;  o = S^T q        (S is [key, value])
  window:   key j is seen from i when j <= i and (i - j < W or j < F)
  sink:     p_j = exp(z_j - M) / (exp(z0 - M) + sum_j exp(z_j - M)), z0 a number per head without a value

`rnd` (optional) is applied where a bfloat16 engine stores a tensor; with rnd=None all is `real`
(float32 by default, float64 to measure float32's own noise).
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


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


# ----------------------------------------------------------------- mechanisms, one function each

def run_order(n_layers, loop):
    """Layer indices in the order they run: layers [start, stop) are passed `times` times, then the rest."""
    if not loop:
        return list(range(n_layers))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n_layers))


def embedding(tokens, table, scale, bigram=None, hashing=None):
    """x_i = table[t_i] * scale (+ bigram[(t_{i-1} * mul_prev + t_i * mul_cur) mod buckets]; row `buckets` for i = 0)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    x = table[tokens] * table.dtype.type(scale)
    if bigram is not None:
        n = hashing["buckets"]
        rows = np.empty(len(tokens), dtype=np.int64)
        rows[0] = n
        rows[1:] = (tokens[:-1] * hashing["mul_prev"] + tokens[1:] * hashing["mul_cur"]) % n
        x = x + bigram[rows]
    return x


def norm_one_plus(x, w, eps):
    r = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + x.dtype.type(eps))
    return x * r * (1 + w)


def norm_plain(x, w, eps):
    r = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + x.dtype.type(eps))
    return x * r * w


def streams_read(X, a):
    """u = sum_s a[s] X[s]; X is [s, T, d]."""
    return np.tensordot(a, X, axes=(0, 0))


def streams_write(X, y, M, c, m):
    """X'[t] = sum_s M[s, t] X[s] + m c[t] y, all t from the old X."""
    return np.tensordot(M.T, X, axes=(1, 0)) + (X.dtype.type(m) * c)[:, None, None] * y[None]


def short_convolution(x, w):
    """y[i, c] = sum_j w[c, j] x[i - (taps - 1 - j), c], zeros before the start; x [T, C], w [C, taps]."""
    T, taps = x.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1]), dtype=x.dtype), x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j][None, :]
    return y


def unit_vectors(x):
    """Each row of the last axis divided by sqrt(sum(x^2) + 1e-6)."""
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + x.dtype.type(1e-6))


def delta_recurrence(q, k, v, g, b):
    """q, k, g [T, H, K]; v [T, H, V]; b [T, H] -> o [T, H, V]. The state starts at zero."""
    T, H, K = q.shape
    V = v.shape[-1]
    S = np.zeros((H, K, V), dtype=q.dtype)
    o = np.zeros((T, H, V), dtype=q.dtype)
    for i in range(T):
        S = S * g[i][:, :, None]
        seen = np.einsum("hkv,hk->hv", S, k[i])
        e = b[i][:, None] * (v[i] - seen)
        S = S + k[i][:, :, None] * e[:, None, :]
        o[i] = np.einsum("hkv,hk->hv", S, q[i])
    return o


def channel_delta(h, p, c, eps, real, rnd=None):
    """The gated delta-rule mixer with a decay per key channel. p: the mixer's tensors by their short names."""
    T = h.shape[0]
    H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    lin = lambda x, name: _keep(rnd, x @ p[name].T)
    q = _keep(rnd, silu(short_convolution(lin(h, "q"), p["q.conv"]))).reshape(T, G, K)
    k = _keep(rnd, silu(short_convolution(lin(h, "k"), p["k.conv"]))).reshape(T, G, K)
    v = _keep(rnd, silu(short_convolution(lin(h, "v"), p["v.conv"]))).reshape(T, H, V)
    q = unit_vectors(q) * real(K) ** real(-0.5)
    k = unit_vectors(k)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(lin(h, "b"))
    step = softplus(lin(h, "a1") @ p["a2"].T + p["dt_bias"]).reshape(T, H, K)
    g = np.exp(-np.exp(p["A_log"])[None, :, None] * step)
    o = delta_recurrence(q, k, v, g, beta)
    o = norm_plain(o, p["norm"], eps)
    gate = sigmoid(lin(h, "g1") @ p["g2"].T).reshape(T, H, V)
    return _keep(rnd, (o * gate).reshape(T, H * V)) @ p["o"].T


def rotate_half_layout(x, positions, base, dims, real):
    """x [T, H, D]: dimension i pairs with i + dims/2, i < dims/2, angle p * base^(-2i/dims); the rest passes."""
    half = dims // 2
    f = real(base) ** (-(np.arange(half, dtype=real) * 2) / real(dims))
    a = np.asarray(positions, dtype=real)[:, None] * f[None, :]
    cos, sin = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def visible(T, window, keep_first):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def softmax_with_sink(z, sink, mask):
    """z [H, T, T] scores, sink [H]; rows sum to less than one by the sink's share."""
    z = np.where(mask[None], z, -np.inf)
    top = np.maximum(z.max(axis=-1), sink[:, None])
    e = np.exp(z - top[..., None])
    return e / (e.sum(axis=-1) + np.exp(sink[:, None] - top))[..., None]


def attention(h, p, c, eps, real, rnd=None):
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    lin = lambda x, name: _keep(rnd, x @ p[name].T)
    q, k, v = lin(h, "q").reshape(T, H, D), lin(h, "k").reshape(T, G, D), lin(h, "v").reshape(T, G, V)
    q, k = norm_plain(q, p["q.norm"], eps), norm_plain(k, p["k.norm"], eps)
    pos = np.arange(T)
    if c.get("rot"):
        q = rotate_half_layout(q, pos, c["rot"]["base"], c["rot"]["dims"], real)
        k = rotate_half_layout(k, pos, c["rot"]["base"], c["rot"]["dims"], real)
    q, k = _keep(rnd, q), _keep(rnd, k)
    rep = H // G
    k, v = np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1)
    z = np.einsum("ihd,jhd->hij", q, k) * real(c["scale"])
    mask = visible(T, c["mask"]["size"], c["mask"]["keep_first"]) if c.get("mask") else visible(T, T, 0)
    w = softmax_with_sink(z, p["sink"].astype(real), mask)
    o = np.einsum("hij,jhv->ihv", w, v).reshape(T, H * V)
    return _keep(rnd, o) @ p["o"].T


def gated_feed_forward(h, p, rnd=None):
    gate, up = _keep(rnd, h @ p["gate"].T), _keep(rnd, h @ p["up"].T)
    return _keep(rnd, silu(gate) * up) @ p["down"].T


# ----------------------------------------------------------------- the model

def forward(config, tensors, tokens, real=np.float32, rnd=None, layers_out=None):
    """Logits [T, vocab] for one sequence from position 0. layers_out: a list that receives the stream (the sum of
    the streams) after every layer run."""
    W = {n: (t.astype(real) if t.dtype.kind == "f" else t) for n, t in tensors.items()}
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    emb = config.get("embedding", {})
    x = embedding(tokens, W["embed"], emb.get("scale", 1.0), W.get("bigram") if emb.get("bigram") else None,
                  emb.get("bigram"))
    s = config.get("streams")
    X = np.stack([x] * s) if s else None
    for l in run_order(len(config["layers"]), config.get("loop")):
        layer = config["layers"][l]
        pre = f"l{l}."
        for q, kind in ((1, "mixer"), (2, "mlp")):
            if layer[kind] is None:
                continue
            u = streams_read(X, W[f"{pre}hc{q}.in"]) if s else x
            hn = _keep(rnd, norm_one_plus(u, W[f"{pre}norm{q}"], eps))
            if kind == "mixer":
                p = {n[len(pre) + 4:]: t for n, t in W.items() if n.startswith(pre + "mix.")}
                fn = {"channel_delta": channel_delta, "attention": attention}[layer["type"]]
                y = fn(hn, p, layer["mixer"], eps, real, rnd)
            else:
                p = {n[len(pre) + 4:]: t for n, t in W.items() if n.startswith(pre + "mlp.")}
                y = gated_feed_forward(hn, p, rnd)
            if s:
                X = streams_write(X, y, W[f"{pre}hc{q}.mix"], W[f"{pre}hc{q}.out"], m)
            else:
                x = x + real(m) * y
        if layers_out is not None:
            layers_out.append((X.sum(axis=0) if s else x).copy())
    if s:
        x = X.sum(axis=0)
    return _keep(rnd, norm_one_plus(x, W["final.norm"], eps)) @ W["head"].T
