"""The retention mixer: linear attention with one fixed decay per head, no softmax and no denominator.

    q = Wq h, k = Wk h   (heads x dim);   v = Wv h   (heads x vdim);   no biases
    the first R dims of every head of q and k are rotated by position * f_i (a `rope` position part: halves pairing,
    dim i with dim i + R/2); k is multiplied by dim^-1/2 after the rotation
    per head and token:  S <- decay_h S + k v^T;  o = S^T q
    out = Wo concat_h (o_h / sqrt(mean(o_h^2) + eps) * silu(Wg h)_h)

The layer keeps nothing per position; per request it keeps S (heads, vdim, dim) in float32, zeroed when a request takes
its state slot.  A step: one product of the mixer's input (q, k, v and the gate side by side), one kernel that rotates
and leaves q, k, v in float32, the recurrence (a sequence's tokens in order, whatever their number: prompts, portions and
single tokens; long stretches cut into segments that run side by side), the gated norm of its output,
the output product.  Angles, the state, the recurrence and the norm are float32.
"""
from ..cache.manager import StateNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import PartSpec, make, register


class Retention:
    def __init__(self, hidden, heads, dim, vdim, decay, eps, position=None, prefix="", names=None):
        self.D, self.H, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.H:
            raise ConfigError(f"{len(self.decay_values)} decays for {heads} heads")
        self.eps = float(eps)
        self.position = make("position", position) if isinstance(position, PartSpec) else position
        n = dict(q="q", k="k", v="v", g="g", o="o")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.state_offset = 0
        self.w_in = self.wo = self.decay = None

    @property
    def graph_safe(self):
        """forward() depends on the batch only through the lengths of the step's arrays; so must the position encoding"""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def wants(self):
        H, D = self.H, self.D
        out = [Want(self.n["q"], (H * self.dim, D), "matrix"), Want(self.n["k"], (H * self.dim, D), "matrix"),
               Want(self.n["v"], (H * self.vdim, D), "matrix"), Want(self.n["g"], (H * self.vdim, D), "matrix"),
               Want(self.n["o"], (D, H * self.vdim), "matrix")]
        return out + (self.position.wants() if self.position is not None else [])

    def bind(self, tensors, env):
        import torch
        t = lambda k: tensors[self.n[k]]
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], 0).contiguous()
        self.wo = t("o")
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=env.device)
        if self.position is not None:
            self.position.bind(tensors, env)
            rot = self.position.rotation()
            if rot is None or rot[2] != 1 or rot[1] > self.dim or rot[1] % 2:
                raise ConfigError("retention rotates the first dims of a head in halves; its position part must do that")

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
        rows = ctx.ws.get("retention_in", N, (self.w_in.shape[0],), ctx.dtype)
        ops.linear(h, self.w_in, out=rows)
        f32 = torch.float32
        q = ctx.ws.get("retention_q", N, (H * dim,), f32)
        k = ctx.ws.get("retention_k", N, (H * dim,), f32)
        v = ctx.ws.get("retention_v", N, (H * vdim,), f32)
        freqs, rd = (None, 0)
        if self.position is not None:
            freqs, rd, _ = self.position.rotation()
        ops.retention_prep(rows, 0, H * dim, 2 * H * dim, ctx.dev("positions"), freqs, q, k, v, H, dim, vdim, rd,
                           dim ** -0.5)
        o = ctx.ws.get("retention_o", N, (H * vdim,), f32)
        off = self.state_offset
        state = ctx.cache.state[run.state_id][:, off:off + self.state_floats()]
        # the number of tokens per sequence follows from the lengths of the step's arrays (N tokens, S sequences)
        chunked = ops.retention_splits(N, ctx.S, H, vdim) and not ctx.options.get("retention_scan_only", False)
        carry = None
        if chunked:             # a row per segment, each a whole state: reserved for the largest step's segments, not its tokens
            carry = ctx.ws.get("retention_carry", ops.retention_carry_rows(N, ctx.S), (H * vdim * dim,), f32,
                               reserve=ops.retention_carry_rows(ctx.ws.max_rows, ctx.S))
        ops.retention(q, k, v, self.decay, o, state, (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("state_slot")), H, dim,
                      vdim, chunked=chunked, carry=carry)
        a = ctx.ws.get("retention_gated", N, (H * vdim,), ctx.dtype)
        ops.gated_rms(o, rows[:, 2 * H * dim + H * vdim:], None, a, H, vdim, self.eps, silu=True)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.linear(a, self.wo, out=y)
        return y, None


register("mixer", "retention", Retention)
