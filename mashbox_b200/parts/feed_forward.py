"""Dense SwiGLU feed-forward: (silu(h Wg^T) * (h Wu^T)) Wd^T, silu and the product in float32
(src/mashbox/gguf/archs/dense.py:356-357).  Gate and up weights are concatenated at load so one product makes both."""
import math

from ..weights.loader import Want
from .base import register


class SwiGLU:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, hidden, intermediate, prefix="", names=None):
        self.D, self.F = int(hidden), int(intermediate)
        n = dict(gate="ffn_gate", up="ffn_up", down="ffn_down")
        n.update(names or {})
        self.names = {k: prefix + v + ".weight" for k, v in n.items()}
        self.wgu = self.wd = None

    def wants(self):
        return [Want(self.names["gate"], (self.F, self.D), "matrix"), Want(self.names["up"], (self.F, self.D), "matrix"),
                Want(self.names["down"], (self.D, self.F), "matrix")]

    def bind(self, tensors, env):
        import torch
        self.wgu = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], 0).contiguous()
        self.wd = tensors[self.names["down"]]

    fuses_small = True      # forward() takes normed= and residual= (see PreNormBlock)

    def forward(self, ctx, h, normed=None, residual=None, out="delta"):
        """out: the workspace buffer the result is left in (a part that runs this one beside something else names
        another one than the default)"""
        import torch
        N = ctx.N
        a = ctx.ws.get("ffn_act", N, (self.F,), ctx.dtype)
        if normed is not None:
            x, norm = normed
            w, eps = norm.fusable()
            ctx.ops.linear_small_normed(x, w, eps, self.wgu, a, "swiglu", held=ctx.take_held(x, norm))
        elif ctx.dtype == torch.bfloat16 and ctx.ops.fused_swiglu_supports(N, self.F, self.D):
            ctx.ops.linear_swiglu(h, self.wgu, a)           # both products and the gate in one kernel
        else:
            gu = ctx.ws.get("gate_up", N, (2 * self.F,), ctx.dtype)
            ctx.ops.linear(h, self.wgu, out=gu)
            ctx.ops.swiglu(gu, a)
        if residual is not None:
            ctx.add_into_stream(a, self.wd, residual)
            return None
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ctx.ops.linear(a, self.wd, out=y)
        return y, None


register("feed_forward", "swiglu", SwiGLU)


def _softplus(t):
    return max(t, 0.0) + math.log1p(math.exp(-abs(t)))


class DenseXielu:
    """act(h Wu^T) Wd^T with the xIELU activation: act(z) = ap z^2 + z/2 for z > 0 and an (e^z - 1 - z) + z/2 otherwise,
    ap = softplus(p), an = 1/2 + softplus(q); the layer's two numbers (p, q) are one stored tensor.  The activation is
    float32 arithmetic on the product's outputs."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, intermediate, prefix="", names=None):
        self.D, self.F = int(hidden), int(intermediate)
        n = dict(up="ffn_up.weight", down="ffn_down.weight", act="ffn_act")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.wu = self.wd = self.ap = self.an = None

    def wants(self):
        return [Want(self.names["up"], (self.F, self.D), "matrix"), Want(self.names["down"], (self.D, self.F), "matrix"),
                Want(self.names["act"], (2,), "vector")]

    def bind(self, tensors, env):
        self.wu, self.wd = tensors[self.names["up"]], tensors[self.names["down"]]
        p, q = (float(v) for v in tensors[self.names["act"]].double().cpu())
        self.ap, self.an = _softplus(p), 0.5 + _softplus(q)

    def forward(self, ctx, h, out="delta"):
        """out: the workspace buffer the result is left in (a block that runs this part beside its mixer names another
        one than the mixer's)"""
        import torch
        N = ctx.N
        a = ctx.ws.get("ffn_act", N, (self.F,), ctx.dtype)
        if ctx.dtype == torch.bfloat16 and ctx.ops.fused_xielu_supports(N, self.F, self.D):
            ctx.ops.linear_xielu(h, self.wu, a, self.ap, self.an)       # the product with the activation in its epilogue
        else:
            z = ctx.ws.get("ffn_up", N, (self.F,), ctx.dtype)
            ctx.ops.linear(h, self.wu, out=z)
            ctx.ops.xielu(z, a, self.ap, self.an)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ctx.ops.linear(a, self.wd, out=y)
        return y, None


register("feed_forward", "dense_xielu", DenseXielu)


class ClampedGLU:
    """Wd (g sigmoid(alpha g) (u + shift)) with g = min(Wg h, limit) -- clamped from above only -- and
    u = clamp(Wu h, -limit, limit): the routed experts' unit as a dense layer.  limit None: no clamps.  Gate and up weights
    are concatenated at load so one product makes both; the activation is float32 arithmetic on the product's outputs."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, intermediate, limit=None, alpha=1.702, shift=1.0, prefix="", names=None):
        self.D, self.F = int(hidden), int(intermediate)
        self.limit = float(limit) if limit else None
        self.alpha, self.shift = float(alpha), float(shift)
        n = dict(gate="ffn_gate", up="ffn_up", down="ffn_down")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.wgu = self.wd = None

    def wants(self):
        return [Want(self.names["gate"], (self.F, self.D), "matrix"), Want(self.names["up"], (self.F, self.D), "matrix"),
                Want(self.names["down"], (self.D, self.F), "matrix")]

    def bind(self, tensors, env):
        import torch
        self.wgu = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], 0).contiguous()
        self.wd = tensors[self.names["down"]]

    def forward(self, ctx, h, out="delta"):
        import torch
        N = ctx.N
        a = ctx.ws.get("ffn_act", N, (self.F,), ctx.dtype)
        if ctx.dtype == torch.bfloat16 and ctx.ops.fused_xielu_supports(N, self.F, self.D) and h.is_contiguous():
            ctx.ops.linear_glu_clamped(h, self.wgu, a, self.limit, self.alpha, self.shift)      # the gate in the product's epilogue
        else:
            gu = ctx.ws.get("gate_up", N, (2 * self.F,), ctx.dtype)
            ctx.ops.linear(h, self.wgu, out=gu)
            ctx.ops.glu_clamped(gu, a, self.limit, self.alpha, self.shift)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ctx.ops.linear(a, self.wd, out=y)
        return y, None


register("feed_forward", "glu_clamped", ClampedGLU)
