"""A recurrent mixer: linear attention with a fixed decay per head (config.specs.DecayAttentionSpec).

Per head a float32 state S [key, value], zero at a sequence's start and carried from token to token:
    S <- decay_h S + k v^T;    o = S^T q
with q, k, v the SiLU of their projections. The heads' outputs, side by side, are normed as one row, multiplied by
sigmoid(Wg x) and projected. The mixer keeps no keys: its cache is the state, and its cost per token does not grow.
The state, the recurrence, the norm and the gate's sigmoid are float32 in both number formats.
"""
import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, to_device
from .linear import Linear


def _up8(n):
    return -(-n // 8) * 8


@MIXERS.register("decay_attention")
class DecayAttention:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if not 1 <= s.key_dim <= 256:
            raise ValueError(f"key_dim {s.key_dim}: the recurrence keeps up to 256 key channels a head")
        if len(s.decay) != s.n_heads:
            raise ValueError(f"{len(s.decay)} decays for {s.n_heads} heads")
        self.qk_size, self.v_size = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        # columns of the stacked product: q, k, v, gate, each from a multiple of 8 elements on
        self.at_k = _up8(self.qk_size)
        self.at_v = self.at_k + _up8(self.qk_size)
        self.at_g = self.at_v + _up8(self.v_size)
        self.width = self.at_g + _up8(self.v_size)

    def param_shapes(self):
        s = self.spec
        return {"wq": (self.qk_size, s.hidden), "wk": (self.qk_size, s.hidden), "wv": (self.v_size, s.hidden),
                "wg": (self.v_size, s.hidden), "out_norm": (self.v_size,), "wo": (s.hidden, self.v_size)}

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        stacked = torch.zeros((self.width, s.hidden), dtype=params["wq"].dtype)
        for at, slot in ((0, "wq"), (self.at_k, "wk"), (self.at_v, "wv"), (self.at_g, "wg")):
            stacked[at:at + params[slot].shape[0]] = params[slot]
        self.in_proj = Linear(to_device(stacked, ctx, ctx.dtype))
        self.out_norm = to_device(params["out_norm"], ctx, torch.float32)
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))
        self.decay = torch.tensor([float(d) for d in s.decay], dtype=torch.float64).to(torch.float32).to(ctx.device)

    def step_weights(self):
        return [self.in_proj.weight, self.out_norm, self.o_proj.weight]

    def cache_need(self):
        s = self.spec
        return CacheNeed(states=(("decay_state", (s.n_heads, s.key_dim, s.value_dim), "float32"),))

    def state_bytes(self):
        """Bytes of state a sequence holds in one entry (what a decode step reads and writes for it)."""
        s = self.spec
        return 4 * s.n_heads * s.key_dim * s.value_dim

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if not cache.owns_storage:
            raise ops.KernelRefused("a recurrent entry keeps a state of its own; it cannot read another entry's")
        proj = ws.get("decay_proj", (n, self.width), dt)
        self.in_proj.forward(xn, proj, n)
        o = ws.get("decay_o", (n, self.v_size), torch.float32)
        if batch.is_decode:  # a token a sequence: the recurrence as it stands
            ops.lightning_scan(proj, 0, self.at_k, self.at_v, s.n_heads, s.key_dim, s.value_dim, self.decay,
                               cache.states["decay_state"], o, batch)
        else:  # prompts: in chunks of 64 tokens, only the states between chunks along the sequence
            ops.lightning_chunks(proj, 0, self.at_k, self.at_v, s.n_heads, s.key_dim, s.value_dim, self.decay,
                                 cache.states["decay_state"], o, batch, ws)
        normed = ws.get("decay_normed", (n, self.v_size), dt)
        ops.gated_row_norm(o, proj[:, self.at_g:], self.out_norm, normed, s.norm_eps, batch)
        self.o_proj.forward(normed, out, n)
        return out
