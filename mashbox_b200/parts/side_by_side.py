"""Two mixers side by side: both read the same input.  How their outputs meet is `combine`:

    "mean_of_norms" (the default): each output is RMS-normed over the model width with a weight of its own, and the
        result is half their sum:  out = (left(h) / rms(left(h)) * wl + right(h) / rms(right(h)) * wr) / 2
    "sum": out = left_scale * left(h) + right_scale * right(h), two constants and no tensors.  A block that norms its
        sublayers' outputs takes the two outputs and their weights as they are (`forward_parts`) and sums them in the
        kernel that norms.

`left` and `right` are the specs of any two registered mixers whose forward() takes `out=` (the workspace buffer its
result is left in); their tensors live under `left_prefix` and `right_prefix`, the two weights under `left_weight`
and `right_weight`.  At most one of the two may keep something per position (it owns the run's cache); what they keep
per request is laid side by side in one flat float32 state."""
from ..cache.manager import StateNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import make, register


class SideBySide:
    def __init__(self, hidden, left, right, eps, prefix="", left_prefix="left.", right_prefix="right.",
                 left_weight="left.out", right_weight="right.out", combine="mean_of_norms", left_scale=1.0,
                 right_scale=1.0):
        self.D, self.eps = int(hidden), float(eps)
        if combine not in ("mean_of_norms", "sum"):
            raise ConfigError(f"two mixers side by side cannot be combined by {combine!r}")
        self.combine, self.scales = combine, (float(left_scale), float(right_scale))
        if combine == "sum":
            self.forward_parts = self._forward_parts
        self.left = make("mixer", left, prefix=prefix + left_prefix)
        self.right = make("mixer", right, prefix=prefix + right_prefix)
        self.names = (prefix + left_weight, prefix + right_weight)
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ConfigError("of two mixers side by side only one may keep something per position")
        off = 0
        for part in (self.left, self.right):
            if part.state_need() is not None:
                if not hasattr(part, "state_floats"):
                    raise ConfigError("a mixer side by side with another must say how many floats of state it keeps")
                part.state_offset = off
                off += part.state_floats()
        self.state_total = off
        self.wl = self.wr = None

    @property
    def graph_safe(self):
        return bool(getattr(self.left, "graph_safe", False)) and bool(getattr(self.right, "graph_safe", False))

    def wants(self):
        own = [Want(self.names[0], (self.D,), "vector"), Want(self.names[1], (self.D,), "vector")]
        return self.left.wants() + self.right.wants() + (own if self.combine == "mean_of_norms" else [])

    def bind(self, tensors, env):
        self.left.bind(tensors, env)
        self.right.bind(tensors, env)
        if self.combine == "mean_of_norms":
            self.wl, self.wr = tensors[self.names[0]], tensors[self.names[1]]

    def cache_need(self):
        need = self.left.cache_need()
        return need if need is not None else self.right.cache_need()

    def state_need(self):
        return StateNeed((self.state_total,), "float32") if self.state_total else None

    def prepare(self, ctx):
        self.left.prepare(ctx)
        self.right.prepare(ctx)

    def _forward_parts(self, ctx, h, run):
        """-> (left output, its weight, right output, its weight) for whoever sums them itself"""
        a, bias_a = self.left.forward(ctx, h, run, out="side_left")
        b, bias_b = self.right.forward(ctx, h, run, out="side_right")
        if bias_a is not None or bias_b is not None:
            raise ConfigError("mixers side by side cannot defer a bias")
        return a, self.scales[0], b, self.scales[1]

    def forward(self, ctx, h, run, out="delta"):
        a, sa, b, sb = self._forward_parts(ctx, h, run)
        y = ctx.ws.get(out, ctx.N, (self.D,), ctx.dtype)
        if self.combine == "sum":       # a block that cannot take the parts: two passes, the sum rounded twice
            import torch
            torch.mul(a, sa, out=y)
            y.add_(b, alpha=sb)
            return y, None
        ctx.ops.rms_pair_mean(a, b, self.wl, self.wr, y, self.eps)
        return y, None


register("mixer", "side_by_side", SideBySide)
