"""The Movarax decoder: its name in config.json and the names of its tensors.

Layer i's tensors start with "l<i>."; a mixer's are "l<i>.mix.*", a feed-forward's "l<i>.mlp.*" (expert e's
"l<i>.mlp.e<e>.*", the shared expert's "l<i>.mlp.shared.*"), the two norms "l<i>.norm1" and "l<i>.norm2".
"""
from ..config.movarax import MovaraxConfig
from ..config.registry import register_architecture
from .layout import ModelLayout
from .model import expected_tensors

_LATENT = {"wq": "q", "wdown": "dkv", "down_norm": "dkv.norm", "wuk": "uk", "wuv": "uv", "sink": "sink", "wo": "o"}
_DECAY = {"wq": "q", "wk": "k", "wv": "v", "wg": "g", "out_norm": "norm", "wo": "o"}


class MovaraxArchitecture:
    name = "Movarax"

    def parse_config(self, raw):
        return MovaraxConfig.from_dict(raw)

    def layout(self, spec):
        layers = []
        for l, block in enumerate(spec.layers):
            p = f"l{l}."
            names = {("mixer_norm", "weight"): p + "norm1"}
            table = _LATENT if block.mixer.kind == "latent_attention" else _DECAY
            for slot, short in table.items():
                names[("mixer", slot)] = p + "mix." + short
            ffn = block.ffn
            if ffn is not None:
                names[("ffn_norm", "weight")] = p + "norm2"
                if ffn.kind == "routed_mlp":
                    names[("ffn", "router")] = p + "mlp.router"
                    for e in range(ffn.experts):
                        names[("ffn", f"up{e}")] = f"{p}mlp.e{e}.up"
                        names[("ffn", f"down{e}")] = f"{p}mlp.e{e}.down"
                    names[("ffn", "shared_up")] = p + "mlp.shared.up"
                    names[("ffn", "shared_down")] = p + "mlp.shared.down"
                else:
                    for slot in ("gate", "up", "down"):
                        names[("ffn", slot)] = p + "mlp." + slot
            layers.append(names)
        return ModelLayout(embed="embed", final_norm="final.norm", head="head", layers=layers)

    def random_moments(self, name, shape, std, norm_std):
        """(mean, amplitude) of a random tensor of this design where the general rule (matrices around zero, vectors
        around one) does not fit; None: the general rule."""
        if name.endswith(".sink"):
            return 0.0, 1.0
        return None

    def info(self, spec):
        kinds = "".join("a" if b.mixer.kind == "latent_attention" else "l" for b in spec.layers)
        ffs = "".join("-" if b.ffn is None else "e" if b.ffn.kind == "routed_mlp" else "d" for b in spec.layers)
        return f"movarax dim={spec.hidden} layers={len(spec.layers)} ({kinds}; feed-forwards {ffs}) vocab={spec.vocab}"

    def tensor_names(self, spec, available=None):
        return expected_tensors(spec, self.layout(spec), available)


register_architecture(MovaraxArchitecture())
