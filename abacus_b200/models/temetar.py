"""The Temetar decoder: its name in config.json and the names of its tensors.

Layer i's tensors start with "l<i>."; a mixer's are "l<i>.mix.*", a feed-forward's "l<i>.mlp.*", the two norms
"l<i>.norm1" and "l<i>.norm2", the stream connections of the two branches "l<i>.hc1.*" and "l<i>.hc2.*".
"""
from ..config.registry import register_architecture
from ..config.temetar import TemetarConfig
from .layout import ModelLayout
from .model import expected_tensors

_ATTENTION = {"wq": "q", "wk": "k", "wv": "v", "wo": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
_DELTA = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wb": "b",
          "decay_in": "a1", "decay_out": "a2", "decay_log": "A_log", "decay_bias": "dt_bias", "gate_in": "g1",
          "gate_out": "g2", "out_norm": "norm", "wo": "o"}
_LINK = {"enter": "in", "leave": "out", "mix": "mix"}


class TemetarArchitecture:
    name = "Temetar"

    def parse_config(self, raw):
        return TemetarConfig.from_dict(raw)

    def complete_config(self, config, shapes):
        """Sizes that config.json leaves to the tensors, read from their shapes ({name: shape})."""
        return config.with_ranks(shapes)

    def layout(self, spec):
        layers = []
        for l, block in enumerate(spec.layers):
            p = f"l{l}."
            names = {("mixer_norm", "weight"): p + "norm1"}
            table = _ATTENTION if block.mixer.kind == "attention" else _DELTA
            for slot, short in table.items():
                names[("mixer", slot)] = p + "mix." + short
            if block.ffn is not None:
                names[("ffn_norm", "weight")] = p + "norm2"
                for slot in ("gate", "up", "down"):
                    names[("ffn", slot)] = p + "mlp." + slot
            if block.learned:
                for slot, short in _LINK.items():
                    names[("mixer_link", slot)] = p + "hc1." + short
                    if block.ffn is not None:
                        names[("ffn_link", slot)] = p + "hc2." + short
            layers.append(names)
        return ModelLayout(embed="embed", final_norm="final.norm", head="head", layers=layers, frame={"pairs": "bigram"})

    def random_moments(self, name, shape, std, norm_std):
        """(mean, amplitude) of a random tensor of this design where the general rule (matrices around zero, vectors
        around one) would not give a model that runs sensibly; None: the general rule."""
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            return 0.0, norm_std                      # stored around zero
        if ".hc" in name:
            s = shape[0]
            return {"in": (1.0 / s, 0.1 / s), "out": (1.0, 0.1), "mix": (1.0 / s, 0.1 / s)}[last]
        if last in ("A_log", "dt_bias"):
            return 0.0, 0.5
        if last == "sink":
            return 0.0, 1.0
        if last == "conv":
            return 0.3, 0.3
        return None

    def info(self, spec):
        kinds = "".join("a" if b.mixer.kind == "attention" else "d" for b in spec.layers)
        return (f"temetar dim={spec.hidden} layers={len(spec.layers)} ({kinds}) runs={len(spec.schedule)} "
                f"streams={spec.frame_spec.streams} vocab={spec.vocab}")

    def tensor_names(self, spec, available=None):
        return expected_tensors(spec, self.layout(spec), available)


register_architecture(TemetarArchitecture())
