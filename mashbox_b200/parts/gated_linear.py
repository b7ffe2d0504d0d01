"""Gated linear attention: a recurrent layer whose state is a matrix per head, decayed per key channel, without a delta
step and without a softmax.

    q = Wq h * dim^-1/2, k = Wk h   (heads x dim);   v = Wv h   (heads x vdim);   no biases
    a = sigmoid(Wa2 (Wa1 h) + ba)^(1/tau)           (heads x dim: one decay per head and key channel, in (0, 1))
    per head and token:  S <- diag(a) S + k v^T;  o = S^T q
    out = Wo concat_h (o_h / sqrt(mean(o_h^2) + eps) * n * silu(Wg h)_h)          n: vdim values, shared by the heads

The layer keeps nothing per position; per request it keeps S (heads, dim, vdim) in float32, zeroed when a request takes
its state slot.  A step: one product of the mixer's input (q, k, v and the gate side by side), the two narrow products of
the decay (the second leaves float32 logits), one kernel that leaves q, k, v and the decays in float32, the recurrence
(the kernel of the delta rule without its delta step: a sequence's tokens in order, whatever their number), the gated
norm of its output, the output product.  The decays -- logarithm of the sigmoid, division by tau, exponential --, the
state, the recurrence and the norm are float32.
"""
from ..cache.manager import StateNeed
from ..weights.loader import Want
from .base import register


class GatedLinearAttention:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, heads, dim, vdim, tau, eps, decay_rank=None, prefix="", names=None):
        self.D, self.H, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.tau, self.eps = float(tau), float(eps)
        self.decay_rank = int(decay_rank) if decay_rank else -1        # None: whatever the stored tensors have
        n = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a2_bias="a2.b")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.state_offset = 0
        self.w_in = self.wa1 = self.wa2 = self.ba = self.norm_w = self.wo = None

    def wants(self):
        H, D = self.H, self.D
        return [Want(self.n["q"], (H * self.dim, D), "matrix"), Want(self.n["k"], (H * self.dim, D), "matrix"),
                Want(self.n["v"], (H * self.vdim, D), "matrix"), Want(self.n["g"], (H * self.vdim, D), "matrix"),
                Want(self.n["o"], (D, H * self.vdim), "matrix"), Want(self.n["norm"], (self.vdim,), "vector"),
                Want(self.n["a1"], (self.decay_rank, D), "matrix"), Want(self.n["a2"], (H * self.dim, self.decay_rank), "matrix"),
                Want(self.n["a2_bias"], (H * self.dim,), "vector")]

    def bind(self, tensors, env):
        import torch

        from ..errors import ConfigError
        t = lambda k: tensors[self.n[k]]
        if t("a1").shape[0] != t("a2").shape[1]:
            raise ConfigError("the two matrices of the decay's low-rank product do not fit each other")
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], 0).contiguous()
        self.wa1, self.wa2, self.ba = t("a1"), t("a2"), t("a2_bias")
        self.norm_w, self.wo = t("norm"), t("o")

    def cache_need(self):
        return None

    def state_floats(self):
        return self.H * self.dim * self.vdim

    def state_need(self):
        return StateNeed((self.state_floats(),), "float32")

    def prepare(self, ctx):
        pass

    def forward(self, ctx, h, run, out="delta"):
        import torch
        ops, N = ctx.ops, ctx.N
        H, dim, vdim = self.H, self.dim, self.vdim
        f32 = torch.float32
        rows = ctx.ws.get("gla_in", N, (self.w_in.shape[0],), ctx.dtype)
        ops.linear(h, self.w_in, out=rows)
        low = ctx.ws.get("gla_low", N, (self.wa1.shape[0],), ctx.dtype)
        ops.linear(h, self.wa1, out=low)
        z = ctx.ws.get("gla_z", N, (H * dim,), f32)
        ops.linear(low, self.wa2, out=z, out_dtype=f32)
        q = ctx.ws.get("gla_q", N, (H * dim,), f32)
        k = ctx.ws.get("gla_k", N, (H * dim,), f32)
        v = ctx.ws.get("gla_v", N, (H * vdim,), f32)
        g = ctx.ws.get("gla_g", N, (H * dim,), f32)
        ops.gla_gates(rows, z, self.ba, self.tau, q, k, v, g, H, dim, vdim)
        o = ctx.ws.get("gla_o", N, (H * vdim,), f32)
        off = self.state_offset
        state = ctx.cache.state[run.state_id][:, off:off + self.state_floats()]
        ops.gated_scan(q, k, v, g, o, state, (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("state_slot")), H, H, dim, vdim,
                       per_head=False)
        a = ctx.ws.get("gla_gated", N, (H * vdim,), ctx.dtype)
        ops.gated_rms(o, rows[:, 2 * H * dim + H * vdim:], self.norm_w, a, H, vdim, self.eps, silu=True)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.linear(a, self.wo, out=y)
        return y, None


register("mixer", "gla", GatedLinearAttention)
