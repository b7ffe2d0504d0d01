"""The state-space-duality mixer: a recurrent layer whose state is a matrix per head with ONE decay per head and token,
behind a short causal convolution.

    Win h = [z | x | B | C | dt]: z, x inner = heads * vdim wide; B, C groups * state wide (head h reads group
    h // (heads / groups)); dt one number per head
    (x, B, C) <- silu(conv(x, B, C) + conv bias): a causal filter of `taps` per channel, zeros before the start
    dt <- softplus(dt + dt_bias)   (no clamp)
    per head and token:  S <- exp(-exp(A_log_h) dt) S + dt B x^T   (S: state x vdim);   y = S^T C + D_h x
    out = Wo (rms over each of `norm_groups` equal stretches of (y * silu(z)), times n)       the gate BEFORE the norm

The layer keeps nothing per position; per request it keeps one flat float32 state: the last taps - 1 rows of (x, B, C)
before the convolution (`parts/conv.py`'s layout), then S (heads, state, vdim).  A slot is zeroed when a request takes
it.  A step: three products of the mixer's input ((x, B, C); z; dt, which leaves float32), the convolution kernel, one
kernel that makes everything the recurrence reads in float32 (B is its key, C its query, dt x its value, so the state
takes in dt B x^T), the recurrence (the kernel of the gated scans with one decay per head), one kernel for skip, gate,
grouped norm and weight, the output product.  dt, softplus, the decay and its exponentials, the state, the recurrence
and the norm are float32.
"""
from ..cache.manager import StateNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import register
from .conv import plan_sequences, state_view, step_sequences


class StateSpaceDuality:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, heads, vdim, state, eps, groups=1, norm_groups=1, taps=1, prefix="", names=None):
        self.D, self.H, self.P, self.NS = int(hidden), int(heads), int(vdim), int(state)
        self.G, self.parts_n, self.taps, self.eps = int(groups or 1), int(norm_groups or 1), int(taps or 1), float(eps)
        if self.G < 1 or self.H % self.G:
            raise ConfigError(f"{heads} heads do not divide into {groups} groups")
        self.inner = self.H * self.P
        if self.inner % self.parts_n:
            raise ConfigError(f"{norm_groups} norm groups do not divide {self.inner} channels")
        self.C = self.inner + 2 * self.G * self.NS          # the channels that pass the convolution
        n = dict(w_in="in", conv="conv", conv_bias="conv.b", dt="dt_bias", A="A_log", D="D", norm="norm", o="o")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.state_offset = 0
        self.w_xbc = self.w_z = self.w_dt = self.wconv = self.cb = self.dt_bias = self.A = self.Dw = self.norm_w = self.wo = None

    def wants(self):
        return [Want(self.n["w_in"], (2 * self.inner + 2 * self.G * self.NS + self.H, self.D), "matrix"),
                Want(self.n["conv"], (self.C, self.taps), "vector"), Want(self.n["conv_bias"], (self.C,), "vector"),
                Want(self.n["dt"], (self.H,), "vector"), Want(self.n["A"], (self.H,), "vector"),
                Want(self.n["D"], (self.H,), "vector"), Want(self.n["norm"], (self.inner,), "vector"),
                Want(self.n["o"], (self.D, self.inner), "matrix")]

    def bind(self, tensors, env):
        t = lambda k: tensors[self.n[k]]
        w = t("w_in")
        self.w_z = w[:self.inner].contiguous()
        self.w_xbc = w[self.inner:self.inner + self.C].contiguous()
        self.w_dt = w[self.inner + self.C:].contiguous()
        self.wconv = t("conv").t().contiguous()             # (taps, channels), as the kernels read them
        self.cb, self.dt_bias, self.A, self.Dw, self.norm_w, self.wo = (t("conv_bias"), t("dt"), t("A"), t("D"), t("norm"),
                                                                       t("o"))

    def cache_need(self):
        return None

    def conv_floats(self):
        return (self.taps - 1) * self.C

    def state_floats(self):
        return self.conv_floats() + self.H * self.NS * self.P

    def state_need(self):
        return StateNeed((self.state_floats(),), "float32")

    def prepare(self, ctx):
        plan_sequences(ctx)

    def forward(self, ctx, h, run, out="delta"):
        import torch
        ops, N = ctx.ops, ctx.N
        H, G, P, NS = self.H, self.G, self.P, self.NS
        f32 = torch.float32
        xbc = ctx.ws.get("ssd_xbc", N, (self.C,), ctx.dtype)
        ops.linear(h, self.w_xbc, out=xbc)
        z = ctx.ws.get("ssd_z", N, (self.inner,), ctx.dtype)
        ops.linear(h, self.w_z, out=z)
        dt = ctx.ws.get("ssd_dt", N, (H,), f32)
        ops.linear(h, self.w_dt, out=dt, out_dtype=f32)
        conv = ctx.ws.get("ssd_conv", N, (self.C,), ctx.dtype)      # a filter of one tap keeps no state
        ops.short_conv(xbc, self.wconv, state_view(ctx, run.state_id, self.state_offset, self.taps, self.C),
                       step_sequences(ctx), conv)
        xbc = conv
        q = ctx.ws.get("ssd_q", N, (G * NS,), f32)
        k = ctx.ws.get("ssd_k", N, (G * NS,), f32)
        v = ctx.ws.get("ssd_v", N, (self.inner,), f32)
        g = ctx.ws.get("ssd_g", N, (H,), f32)
        ops.ssd_gates(xbc, self.cb, dt, self.dt_bias, self.A, q, k, v, g, H, G, P, NS)
        o = ctx.ws.get("ssd_o", N, (self.inner,), f32)
        off = self.state_offset + self.conv_floats()
        state = ctx.cache.state[run.state_id][:, off:off + H * NS * P]
        ops.gated_scan(q, k, v, g, o, state, (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("state_slot")), H, G, NS, P,
                       per_head=True)
        a = ctx.ws.get("ssd_gated", N, (self.inner,), ctx.dtype)
        ops.ssd_out(o, xbc, self.cb, self.Dw, z, self.norm_w, a, H, P, self.parts_n, self.eps)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.linear(a, self.wo, out=y)
        return y, None


register("mixer", "ssd", StateSpaceDuality)
