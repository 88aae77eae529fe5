"""Typed configuration of the Temetar decoder, read from config.json.

A Temetar model is a list of layers that may differ one from the next: each has a mixer, either attention (grouped
heads with values of their own size, a norm of q and k per head, rotary positions on part of a head, a sliding window
that also keeps the sequence's first keys, a sink in the softmax) or a gated delta rule with a decay per key channel,
and an optional gated feed-forward. The residual stream is kept as several copies with learned connections, the
embedding is scaled and joined by a table hashed on token pairs, and a range of layers may run several times in a
row with the same weights, each pass with a cache or state of its own. Every size and constant comes from
config.json (or, for the inner sizes of the delta rule's decay and gate, from the tensors' shapes).
"""
import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import ConfigError
from .specs import (AttentionSpec, DeltaRuleSpec, GatedMLPSpec, ModelSpec, NormSpec, PairEmbeddingSpec, RotarySpec,
                    ScheduleEntry, StreamsBlockSpec)

MAX_POSITIONS = 1 << 20  # the design has no limit of its own; the engine's cache sets the real one


def _int(where, raw, key, minimum=1, default=None):
    v = raw.get(key, default) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _float(where, raw, key, default=None, positive=True):
    v = raw.get(key, default) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class TemetarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: Optional[float]   # None: no rotation
    rot_dims: int
    window: Optional[int]       # None: every earlier key
    keep_first: int

    @classmethod
    def from_dict(cls, where, m):
        heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: {where}heads {heads} is no multiple of kv_heads {kv}")
        dim = _int(where, m, "dim")
        rot, mask = m.get("rot"), m.get("mask")
        base, dims = None, 0
        if rot is not None:
            base, dims = _float(where + "rot.", rot, "base"), _int(where + "rot.", rot, "dims", 2)
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most dim {dim}")
        window, keep = None, 0
        if mask is not None:
            window = _int(where + "mask.", mask, "size")
            keep = _int(where + "mask.", mask, "keep_first", 0, 0)
        return cls(heads, kv, dim, _int(where, m, "vdim", 1, dim), _float(where, m, "scale"), base, dims, window, keep)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_base is not None:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return d


@dataclass(frozen=True)
class TemetarDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = 0   # inner sizes of the decay's and the gate's pairs of matrices: config.json does not carry
    gate_rank: int = 0    # them; they are read from the tensors (0 until then)

    @classmethod
    def from_dict(cls, where, m):
        heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: {where}heads {heads} is no multiple of kv_heads {kv}")
        return cls(heads, kv, _int(where, m, "dim"), _int(where, m, "vdim"), _int(where, m, "conv"),
                   _int(where, m, "decay_rank", 0, 0), _int(where, m, "gate_rank", 0, 0))

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class TemetarLayer:
    type: str                 # "attention" or "channel_delta"
    mixer: object
    ff: Optional[int]         # None: the layer has no feed-forward


@dataclass(frozen=True)
class TemetarConfig:
    vocab: int
    width: int
    layers: Tuple[TemetarLayer, ...]
    eps: float
    residual_mult: float = 1.0
    streams: Optional[int] = None            # None: one stream with the plain residual sum, no connection tensors
    embedding_scale: float = 1.0
    bigram: Optional[Tuple[int, int, int]] = None   # (buckets, mul_prev, mul_cur)
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times)
    architecture: str = "Temetar"

    @classmethod
    def from_dict(cls, raw):
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        parsed = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind == "attention":
                mixer = TemetarAttention.from_dict(where + "mixer.", layer.get("mixer"))
            elif kind == "channel_delta":
                mixer = TemetarDelta.from_dict(where + "mixer.", layer.get("mixer"))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is neither attention nor channel_delta")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind')!r} is not built (only dense)")
            parsed.append(TemetarLayer(kind, mixer, None if mlp is None else _int(where + "mlp.", mlp, "ff")))
        emb = raw.get("embedding") or {}
        big = emb.get("bigram")
        bigram = None
        if big is not None:
            bigram = (_int("embedding.bigram.", big, "buckets"), _int("embedding.bigram.", big, "mul_prev", 0),
                      _int("embedding.bigram.", big, "mul_cur", 0))
        loop = raw.get("loop")
        if loop is not None:
            start, stop = _int("loop.", loop, "start", 0), _int("loop.", loop, "stop", 0)
            times = _int("loop.", loop, "times", 0)
            if not start <= stop <= len(parsed):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(parsed)} layers")
            loop = (start, stop, times)
        streams = raw.get("streams")
        if streams is not None:
            streams = _int("", raw, "streams")
            if streams > 8:
                raise ConfigError(f"config.json: streams {streams}: up to 8 are built")
        return cls(vocab=_int("", raw, "vocab"), width=_int("", raw, "width"), layers=tuple(parsed),
                   eps=_float("norm.", raw.get("norm"), "eps"),
                   residual_mult=_float("", raw, "residual_mult", 1.0, positive=False), streams=streams,
                   embedding_scale=_float("embedding.", emb, "scale", 1.0, positive=False), bigram=bigram, loop=loop)

    def with_ranks(self, shapes):
        """The same configuration with the delta-rule layers' inner sizes read from the tensors' shapes
        ({name: shape}; the second matrices of the decay and of the gate are [.., rank])."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "channel_delta":
                a, g = shapes.get(f"l{i}.mix.a2"), shapes.get(f"l{i}.mix.g2")
                if a is None or g is None or len(a) != 2 or len(g) != 2:
                    raise ConfigError(f"layer {i}: the tensors l{i}.mix.a2 and l{i}.mix.g2 give the inner sizes of the "
                                      "decay and the gate, and are missing")
                m = TemetarDelta(m.heads, m.kv_heads, m.dim, m.vdim, m.conv, int(a[1]), int(g[1]))
            layers.append(TemetarLayer(layer.type, m, layer.ff))
        return TemetarConfig(**{**self.__dict__, "layers": tuple(layers)})

    def to_dict(self):
        """A config.json that from_dict reads back to this object (the inner sizes aside, which the tensors carry)."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "residual_mult": self.residual_mult,
             "embedding": {"scale": self.embedding_scale},
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                         "mlp": None if l.ff is None else {"ff": l.ff, "kind": "dense"}} for l in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.bigram is not None:
            d["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d

    def run_order(self):
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_spec(self):
        norm = NormSpec(self.width, self.eps, one_plus=True)
        streams = self.streams or 1
        blocks = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                rotary = RotarySpec(theta=m.rot_base, rotary_dim=m.rot_dims, pairing="half") if m.rot_base else None
                mixer = AttentionSpec(hidden=self.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                                      scale=m.scale, qk_norm_eps=self.eps, position=rotary, window=m.window,
                                      v_head_dim=m.vdim, keep_first=m.keep_first, sink=True, exact_weights=True)
            else:
                mixer = DeltaRuleSpec(hidden=self.width, n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim,
                                      value_dim=m.vdim, conv_taps=m.conv, decay_rank=max(m.decay_rank, 1),
                                      gate_rank=max(m.gate_rank, 1), norm_eps=self.eps)
            ffn = None if layer.ff is None else GatedMLPSpec(self.width, layer.ff, "silu")
            blocks.append(StreamsBlockSpec(mixer_norm=norm, mixer=mixer, ffn_norm=norm if ffn else None, ffn=ffn,
                                           streams=streams, branch_scale=self.residual_mult,
                                           learned=self.streams is not None))
        buckets, mul_prev, mul_cur = self.bigram or (0, 0, 0)
        return ModelSpec(architecture=self.architecture, hidden=self.width, vocab=self.vocab, layers=tuple(blocks),
                         schedule=tuple(ScheduleEntry(l) for l in self.run_order()), final_norm=norm, tied_head=False,
                         max_positions=MAX_POSITIONS, frame="scaled_pairs",
                         frame_spec=PairEmbeddingSpec(self.embedding_scale, buckets, mul_prev, mul_cur, streams))
