"""RMSNorm with the residual add folded in.

y = v * rsqrt(mean(v^2) + eps) * w with the weight multiplied as stored (src/mashbox/gguf/archs/qwen35.py:343-346),
where v is the residual stream plus the output of the sublayer before (the add of src/mashbox/gguf/archs/dense.py:348,
357, here in float32).  One kernel reads x and the delta once, writes x back and writes y.
"""
from ..errors import ConfigError
from ..weights.loader import Want
from .base import register


class RMSNorm:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, width, eps, name):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight = None

    def wants(self):
        return [Want(self.name, (self.width,), "vector")]

    def bind(self, tensors, env):
        self.weight = tensors[self.name]

    def fusable(self):
        """(weight, eps) for a product kernel that normalises the residual stream itself"""
        return self.weight, self.eps

    def forward(self, ctx, x, pending=None, rows=None):
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get("normed" if rows is None else "normed_rows", n_out, (self.width,), ctx.dtype,
                         reserve=None if rows is None else ctx.options.get("logit_rows", 8))
        delta, bias, *more = pending if pending is not None else (None, None)
        if delta is not None:
            ctx.memo.pop("held", None)         # x changes here: what is held for it no longer describes it
        if more:                                # two sublayers that ran side by side left an output each
            if bias is not None:
                raise ConfigError("two pending outputs cannot be combined with a pending bias")
            ctx.ops.add_rmsnorm_pair(x, delta, more[0], self.weight, None, self.eps, out, None, rows)
        else:
            ctx.ops.add_rmsnorm(x, delta, bias, self.weight, self.eps, out, rows)
        return out

    def forward_pair(self, ctx, x, other, pending=None, conv=None):
        """-> (this norm of x, `other`'s norm of x), x first taking in what is pending ((delta, None) or (delta, None,
        second delta)): for two norms of one width and eps that read the same stream, one kernel and one sum of
        squares.  conv = (filters (taps, width), state view): in a step in which every sequence brings one token the
        kernel also adds the short causal convolution of the first output to it and replaces the state."""
        if other.width != self.width or other.eps != self.eps:
            raise ConfigError("norms with different widths or eps cannot be computed as a pair")
        delta, bias, *more = pending if pending is not None else (None, None)
        if bias is not None:
            raise ConfigError("a pair of norms cannot take a pending bias")
        if delta is not None:
            ctx.memo.pop("held", None)
        a = ctx.ws.get("normed", x.shape[0], (self.width,), ctx.dtype)
        b = ctx.ws.get("normed_side", x.shape[0], (self.width,), ctx.dtype)
        if conv is not None:
            ctx.ops.add_rmsnorm_pair_conv(x, delta, more[0] if more else None, self.weight, other.weight, self.eps, a, b,
                                          conv[0], conv[1], ctx.dev("state_slot"))
        else:
            ctx.ops.add_rmsnorm_pair(x, delta, more[0] if more else None, self.weight, other.weight, self.eps, a, b)
        return a, b


register("norm", "rms", RMSNorm)


class DynamicTanh:
    """y = tanh(alpha v) * w + b, element by element: no mean, no variance, no eps.  alpha is one number, w and b are
    vectors, stored as `<name>.alpha`, `<name>` and `<name>.b`; v is the residual stream plus what is pending, as in
    RMSNorm.  `eps` is accepted and not used, so that a model can hand every norm the same parameters."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, width, name, eps=None):
        self.width, self.name = int(width), name
        self.alpha = self.weight = self.bias = None

    def wants(self):
        return [Want(self.name, (self.width,), "vector"), Want(self.name + ".b", (self.width,), "vector"),
                Want(self.name + ".alpha", (), "vector")]

    def bind(self, tensors, env):
        self.weight, self.bias = tensors[self.name], tensors[self.name + ".b"]
        self.alpha = float(tensors[self.name + ".alpha"].float().cpu())

    def elementwise(self):
        """(alpha, w, b) for a kernel that makes this norm's output while it writes the stream"""
        return self.alpha, self.weight, self.bias

    def forward(self, ctx, x, pending=None, rows=None, out=None):
        """out: where the result goes (default: the workspace's buffer of normed rows); it may be x itself"""
        n_out = x.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = ctx.ws.get("normed" if rows is None else "normed_rows", n_out, (self.width,), ctx.dtype,
                             reserve=None if rows is None else ctx.options.get("logit_rows", 8))
        delta, bias, *more = pending if pending is not None else (None, None)
        if bias is not None:
            raise ConfigError("a Dynamic Tanh norm cannot take a pending bias")
        if delta is not None:
            ctx.memo.pop("held", None)
        ctx.ops.dyt(x, delta, self.alpha, self.weight, self.bias, out, rows, more[0] if more else None)
        return out


register("norm", "dyt", DynamicTanh)


class LayerNorm:
    """y = (v - mean(v)) / sqrt(var(v) + eps) * w + b over a row, var the mean of the squared deviations; w and b are
    stored as `<name>` and `<name>.b`.  As a norm of the stream (`forward`) it is the model's last norm.  As a norm of a
    sublayer's OUTPUT (`add_output`) one kernel norms what the sublayer returned (or a weighted sum of two such
    outputs), adds it into the float32 stream and leaves the new stream in the activation dtype for the next reader."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, width, eps, name):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight = self.bias = None

    def wants(self):
        return [Want(self.name, (self.width,), "vector"), Want(self.name + ".b", (self.width,), "vector")]

    def bind(self, tensors, env):
        self.weight, self.bias = tensors[self.name], tensors[self.name + ".b"]

    def forward(self, ctx, x, pending=None, rows=None, out=None):
        n_out = x.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = ctx.ws.get("normed" if rows is None else "normed_rows", n_out, (self.width,), ctx.dtype,
                             reserve=None if rows is None else ctx.options.get("logit_rows", 8))
        if pending is not None:
            delta, bias, *more = pending
            if bias is not None or more:
                raise ConfigError("a layer norm of the stream takes one pending output without a bias")
            ctx.memo.pop("held", None)
            x.add_(delta)
        ctx.ops.layer_norm(x, rows, self.weight, self.bias, self.eps, out)
        return out

    def add_output(self, ctx, x, y, copy=None, y2=None, s1=1.0, s2=1.0):
        """x += ln(s1 y + s2 y2) w + b; copy: the new x in the activation dtype"""
        ctx.memo.pop("held", None)
        ctx.ops.ln_add(x, y, self.weight, self.bias, self.eps, copy, y2, s1, s2)


register("norm", "layer", LayerNorm)
