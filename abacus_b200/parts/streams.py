"""A layer over a residual stream that is kept as several copies with learned connections
(config.specs.StreamsBlockSpec), and the connection itself as a part.

The stream of a step is X float32 [tokens, s, d]. A branch with connection (enter [s], mix [s, s] indexed
[from, to], leave [s]) and the block's multiplier m reads u = sum_s enter[s] X[s], runs on norm(u), and its
output y is written back as X'[t] = sum_s mix[s, t] X[s] + m leave[t] y for all t at once. As in the pre-norm
block the write is not done where y is made: it is handed on (`Pending`) and done by the kernel that reads for the
next branch (csrc/streams.cu), of this block, of the next one or of the frame's last norm; so the streams are read
and written once between two branches. With one stream and no learned connection this is x += m y.
"""
from dataclasses import dataclass

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, to_device


@dataclass
class Pending:
    """A branch's output that is not yet written to the streams, with what the write needs."""
    y: torch.Tensor      # float32 [tokens, d]
    connection: tuple    # (mix [s, s], leave [s]) float32 on the device
    mult: float


class StreamConnection:
    """How one branch reads from the streams and writes to them. learned False: ones, no tensors."""
    capturable = True

    def __init__(self, streams, learned=True):
        self.streams, self.learned = streams, learned

    def param_shapes(self):
        s = self.streams
        return {"enter": (s,), "leave": (s,), "mix": (s, s)} if self.learned else {}

    def bind(self, params, ctx):
        s = self.streams
        if self.learned:
            self.enter = to_device(params["enter"], ctx, torch.float32)
            self.leave = to_device(params["leave"], ctx, torch.float32)
            self.mix = to_device(params["mix"], ctx, torch.float32)
        else:
            if s != 1:
                raise ValueError("streams without learned connections: only one stream is the plain residual sum")
            self.enter = torch.ones(1, dtype=torch.float32, device=ctx.device)
            self.leave = torch.ones(1, dtype=torch.float32, device=ctx.device)
            self.mix = torch.ones((1, 1), dtype=torch.float32, device=ctx.device)

    def step_weights(self):
        return [self.enter, self.leave, self.mix]


def read_streams(x, pending, enter, norm, out, rows=None, n_rows=None):
    """Write what is pending (if anything), read with `enter`, norm with `norm` (an RMSNorm part; None: no norm)."""
    y, connection, mult = (pending.y, pending.connection, pending.mult) if pending is not None else (None, None, 0.0)
    ops.streams_step(x, y, connection, mult, enter, norm.weight if norm is not None else None,
                     norm.spec.eps if norm is not None else 0.0, out, rows=rows, n_rows=n_rows)
    return out


@BLOCKS.register("streams_pre_norm")
class StreamsBlock:
    def __init__(self, spec):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.mixer_link = StreamConnection(spec.streams, spec.learned)
        self.has_ffn = spec.ffn is not None
        if self.has_ffn:
            self.ffn_norm = NORMS.build(spec.ffn_norm)
            self.ffn = FEED_FORWARDS.build(spec.ffn)
            self.ffn_link = StreamConnection(spec.streams, spec.learned)

    def parts(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_link": self.mixer_link}
        if self.has_ffn:
            parts.update(ffn_norm=self.ffn_norm, ffn=self.ffn, ffn_link=self.ffn_link)
        return parts

    def bind(self, params, ctx):
        """params: {part name: {slot: tensor}}."""
        self.ctx = ctx
        for name, part in self.parts().items():
            part.bind(params[name], ctx)

    def forward(self, x, pending, batch, cache, ws):
        """x float32 [tokens, s, d]; pending: the Pending of the branch before, or None. Returns this block's last."""
        n, d, m = batch.n_rows, x.shape[-1], self.spec.branch_scale
        xn = ws.get("xn", (n, d), self.ctx.dtype)
        read_streams(x, pending, self.mixer_link.enter, self.mixer_norm, xn, n_rows=n)
        # one branch buffer serves: what a Pending holds is read by the next read_streams, which runs (in stream
        # order) before the next branch writes the buffer again
        out = ws.get("branch", (n, d), torch.float32)
        self.mixer.forward(xn, out, batch, cache, ws)
        pending = Pending(out, (self.mixer_link.mix, self.mixer_link.leave), m)
        if self.has_ffn:
            read_streams(x, pending, self.ffn_link.enter, self.ffn_norm, xn, n_rows=n)
            self.ffn.forward(xn, out, batch, ws)
            pending = Pending(out, (self.ffn_link.mix, self.ffn_link.leave), m)
        return pending
