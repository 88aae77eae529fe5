"""Typed configuration of the Movarax decoder, read from config.json.

A Movarax model is a list of pre-norm layers that may differ one from the next. A layer's mixer is either latent
attention (keys and values kept as one low-rank latent row per token that the heads share, with one rotated key part,
a sink in the softmax; a layer may read an earlier layer's latents instead of making its own) or linear attention
with a fixed decay per head (a recurrent layer with a float32 state). Its feed-forward is gated and dense, or a set of
routed experts (sigmoid scores, the weight on the expert's input, squared-ReLU experts, an optional shared expert), or
absent. The embedding is scaled. Every size and constant comes from config.json.
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import ConfigError
from .specs import (DecayAttentionSpec, ExpertSpec, GatedMLPSpec, LatentAttentionSpec, ModelSpec, NormSpec,
                    PairEmbeddingSpec, RotarySpec, RoutedMLPSpec, ScheduleEntry, StreamsBlockSpec)
from .temetar import MAX_POSITIONS, _float, _int

LATENT = "latent_attention"
DECAY_TYPES = ("lightning", "lightning_2")  # two names of one mixer


@dataclass(frozen=True)
class MovaraxLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: Optional[float]    # None: no rotation
    rot_dims: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, where, m):
        rot_dim = _int(where, m, "rot_dim", 0)
        rot = m.get("rot")
        base, dims = None, 0
        if rot is not None:
            base, dims = _float(where + "rot.", rot, "base"), _int(where + "rot.", rot, "dims", 0)
            if dims % 2 or dims > rot_dim:
                raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
        if rot_dim % 2:
            raise ConfigError(f"config.json: {where}rot_dim {rot_dim} must be even")
        kv_from = m.get("kv_from")
        if kv_from is not None:
            kv_from = _int(where, m, "kv_from", 0)
        return cls(_int(where, m, "heads"), _int(where, m, "dim"), rot_dim, _int(where, m, "vdim"), _int(where, m, "kv_rank"),
                   _float(where, m, "scale"), base if dims else None, dims, kv_from)

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale}
        if self.rot_base is not None:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class MovaraxDecay:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, where, m):
        heads = _int(where, m, "heads")
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads:
            raise ConfigError(f"config.json: {where}decay must list one number for each of the {heads} heads")
        values = tuple(_float(where + "decay.", {"v": d}, "v", positive=False) for d in decay)
        return cls(heads, _int(where, m, "dim"), _int(where, m, "vdim"), values)

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class MovaraxDense:
    ff: int

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MovaraxExperts:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]  # None: no shared expert

    @classmethod
    def from_dict(cls, where, m):
        router, expert, shared = m.get("router"), m.get("expert"), m.get("shared")
        experts, top = _int(where + "router.", router, "experts"), _int(where + "router.", router, "top")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top {top} is more than the {experts} experts")
        return cls(experts, top, _int(where + "expert.", expert, "ff"),
                   None if shared is None else _int(where + "shared.", shared, "ff"))

    def to_dict(self):
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class MovaraxLayer:
    type: str               # "latent_attention", "lightning" or "lightning_2"
    mixer: object
    mlp: object             # MovaraxDense, MovaraxExperts or None (no feed-forward)


@dataclass(frozen=True)
class MovaraxConfig:
    vocab: int
    width: int
    layers: Tuple[MovaraxLayer, ...]
    eps: float
    embedding_scale: float = 1.0
    architecture: str = "Movarax"

    @classmethod
    def from_dict(cls, raw):
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        parsed = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind == LATENT:
                mixer = MovaraxLatent.from_dict(where + "mixer.", layer.get("mixer"))
            elif kind in DECAY_TYPES:
                mixer = MovaraxDecay.from_dict(where + "mixer.", layer.get("mixer"))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is none of {LATENT}, {', '.join(DECAY_TYPES)}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp_kind = mlp.get("kind", "dense") if isinstance(mlp, dict) else None
                if mlp_kind == "dense":
                    mlp = MovaraxDense(_int(where + "mlp.", mlp, "ff"))
                elif mlp_kind == "moe":
                    mlp = MovaraxExperts.from_dict(where + "mlp.", mlp)
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp_kind!r} is neither dense nor moe")
            parsed.append(MovaraxLayer(kind, mixer, mlp))
        for i, layer in enumerate(parsed):
            m = layer.mixer
            if layer.type != LATENT or m.kv_from is None:
                continue
            j = m.kv_from
            other = parsed[j].mixer if j < i and parsed[j].type == LATENT else None
            if other is None or other.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from {j} must name an earlier latent_attention "
                                  "layer with latents of its own")
            if (other.kv_rank, other.rot_dim, other.rot_base, other.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                raise ConfigError(f"config.json: layers[{i}] reads the latents of layers[{j}], whose kv_rank, rot_dim or "
                                  "rotation differ from its own")
        emb = raw.get("embedding") or {}
        return cls(vocab=_int("", raw, "vocab"), width=_int("", raw, "width"), layers=tuple(parsed),
                   eps=_float("norm.", raw.get("norm"), "eps"),
                   embedding_scale=_float("embedding.", emb, "scale", 1.0, positive=False))

    def to_dict(self):
        """A config.json that from_dict reads back to this object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale},
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                           for l in self.layers]}

    def to_spec(self):
        norm = NormSpec(self.width, self.eps)
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == LATENT:
                rotary = None
                if m.rot_base is not None:
                    rotary = RotarySpec(theta=m.rot_base, rotary_dim=m.rot_dims, pairing="interleaved", exact_angles=True)
                mixer = LatentAttentionSpec(hidden=self.width, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                                            v_head_dim=m.vdim, rank=m.kv_rank, scale=m.scale, norm_eps=self.eps,
                                            position=rotary, sink=True, shares_latents=m.kv_from is not None)
                schedule.append(ScheduleEntry(i, m.kv_from))
            else:
                mixer = DecayAttentionSpec(hidden=self.width, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                                           decay=m.decay, norm_eps=self.eps)
                schedule.append(ScheduleEntry(i))
            if layer.mlp is None:
                ffn = None
            elif isinstance(layer.mlp, MovaraxDense):
                ffn = GatedMLPSpec(self.width, layer.mlp.ff, "silu")
            else:
                e = layer.mlp
                ffn = RoutedMLPSpec(hidden=self.width, experts=e.experts, top=e.top, expert=ExpertSpec(e.ff),
                                    shared=None if e.shared_ff is None else ExpertSpec(e.shared_ff), score="sigmoid",
                                    weight_on="input")
            blocks.append(StreamsBlockSpec(mixer_norm=norm, mixer=mixer, ffn_norm=norm if ffn else None, ffn=ffn,
                                           streams=1, branch_scale=1.0, learned=False))
        return ModelSpec(architecture=self.architecture, hidden=self.width, vocab=self.vocab, layers=tuple(blocks),
                         schedule=tuple(schedule), final_norm=norm, tied_head=False, max_positions=MAX_POSITIONS,
                         frame="scaled_pairs", frame_spec=PairEmbeddingSpec(scale=self.embedding_scale, streams=1))
