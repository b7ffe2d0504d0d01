"""A feed-forward of many small experts of which every token uses a few, chosen by a router.

    z = Wr h (float32);  s = sigmoid(z);  c = s + correction
    the experts form `groups` equal runs of neighbours; a run is worth the sum of its two largest c; experts outside the
    `keep` best runs cannot be chosen; the `top` largest c are chosen; out = sum over the chosen of s_e expert_e(h)
    expert: g = min(Wg h, limit);  u = clamp(Wu h, -limit, limit);  Wd (g sigmoid(alpha g) (u + 1))

Variants, all constructor parameters: the scores may be softmax(z) over all experts (`score="softmax"`); a run may be
worth its largest c alone (`group_worth="max"`); the weights may be multiplied by a constant (`scale`); the expert may be
the plain gated form Wd (silu(Wg h) * (Wu h)) (`limit=None, alpha=1, shift=0`: no clamps, nothing added to u); and an
expert that every token uses (`shared`: the spec of a feed-forward part, its tensors under `shared_prefix`) may be added,
times sigmoid(w_sg . h) when `shared_gate` names such a row (its logit is one more row of the router's product).

The correction moves the choice only: the weights are the plain scores, not renormalised.  The stored matrices of the
experts (`e0`, `e1`, ...) are stacked at load into (experts, rows, columns) tensors.  A step: the router's product with
a float32 result, one kernel that chooses (a warp per token), the experts, and one kernel that sums a token's places in
order.  The experts of a step of few tokens (and of every float32 step) are one kernel with a block per (token, chosen
expert) pair that streams that expert's three matrices; a bfloat16 step of more tokens sorts the pairs by expert on
the device and runs every expert's rows through tensor-core tiles (gate and up with the activation in the epilogue,
then down), so an expert's matrices are read once per 64 of its rows.  The choice is made on
the device and every launch has a shape that follows from the number of tokens, so steps can be captured in graphs.
"""
from ..errors import ConfigError
from ..weights.loader import Want
from .base import make, register


class RoutedExperts:
    # forward() depends on the batch only through the lengths of the step's arrays (graph_safe, below)

    def __init__(self, hidden, intermediate, experts, top, limit, groups=1, keep=1, alpha=1.702, correction=True,
                 score="sigmoid", group_worth="top2", scale=1.0, shift=1.0, shared=None, shared_prefix="mlp.shared.",
                 shared_gate=None, prefix="", names=None):
        self.D, self.F, self.E, self.top = int(hidden), int(intermediate), int(experts), int(top)
        self.groups, self.keep = int(groups or 1), int(keep or 1)
        self.limit = float(limit) if limit is not None else float("inf")
        self.alpha, self.has_correction = float(alpha), bool(correction)
        if score not in ("sigmoid", "softmax") or group_worth not in ("top2", "max"):
            raise ConfigError(f"routed experts: score {score!r} / group worth {group_worth!r} are not known")
        self.score, self.group_worth, self.scale, self.shift = score, group_worth, float(scale), float(shift)
        self.shared = make("feed_forward", shared, prefix=prefix + shared_prefix) if shared is not None else None
        self.shared_gate = prefix + shared_gate if (shared_gate and self.shared is not None) else None
        if self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ConfigError(f"{experts} experts do not form {groups} equal groups of which {keep} are kept")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ConfigError(f"{top} experts cannot be chosen from {keep} groups of {self.E // self.groups}")
        n = dict(router="mlp.router", correction="mlp.correction", expert="mlp.e{}.", gate="gate", up="up", down="down")
        n.update(names or {})
        self.n = {k: (v if k in ("gate", "up", "down") else prefix + v) for k, v in n.items()}
        self.wr = self.corr = self.wg = self.wu = self.wd = None

    @property
    def graph_safe(self):
        return self.shared is None or bool(getattr(self.shared, "graph_safe", False))

    def _expert(self, e, which):
        return self.n["expert"].format(e) + self.n[which]

    def wants(self):
        out = [Want(self.n["router"], (self.E, self.D), "matrix")]
        if self.has_correction:
            out.append(Want(self.n["correction"], (self.E,), "vector"))
        for e in range(self.E):
            out += [Want(self._expert(e, "gate"), (self.F, self.D), "matrix"),
                    Want(self._expert(e, "up"), (self.F, self.D), "matrix"),
                    Want(self._expert(e, "down"), (self.D, self.F), "matrix")]
        if self.shared is not None:
            out += self.shared.wants()
        if self.shared_gate:
            out.append(Want(self.shared_gate, (1, self.D), "matrix"))
        return out

    def bind(self, tensors, env):
        import torch
        self.wr = tensors[self.n["router"]]
        if self.shared is not None:
            self.shared.bind(tensors, env)
        if self.shared_gate:            # the gate's logit is one more row of the router's product
            self.wr = torch.cat([self.wr, tensors[self.shared_gate]], 0).contiguous()
        self.corr = tensors[self.n["correction"]] if self.has_correction else None
        stack = lambda which: torch.stack([tensors[self._expert(e, which)] for e in range(self.E)], 0).contiguous()
        # (E, 2F, D): every expert's gate rows, then its up rows; the kernels that want them apart take views
        self.wgu = torch.cat([stack("gate"), stack("up")], 1).contiguous()
        self.wg, self.wu, self.wd = self.wgu[:, :self.F], self.wgu[:, self.F:], stack("down")

    def forward(self, ctx, h, out="delta"):
        import torch
        ops, N = ctx.ops, ctx.N
        z = ctx.ws.get("router_logits", N, (self.wr.shape[0],), torch.float32)
        ops.linear(h, self.wr, out=z, out_dtype=torch.float32)
        ids = ctx.ws.get("router_ids", N, (self.top,), torch.int32)
        wts = ctx.ws.get("router_weights", N, (self.top,), torch.float32)
        ops.moe_select(z, self.corr, ids, wts, self.groups, self.keep, experts=self.E, softmax=self.score == "softmax",
                       worth=self.group_worth, scale=self.scale)
        ys = gate = None
        if self.shared is not None:
            ys, _ = self.shared.forward(ctx, h, out="shared_out")
            gate = z[:, self.E:] if self.shared_gate else None
        if ops.moe_tc5_supports(N, self.D, self.F, ctx.dtype) and not ctx.options.get("plain_experts", False):
            T = ops.moe_tc5_tiles(ctx.ws.max_rows, self.top, self.E)
            rows = ctx.ws.get("expert_rows", 128 * T, (self.D,), ctx.dtype, reserve=128 * T)
            act = ctx.ws.get("expert_rows_act", 128 * T, (self.F,), ctx.dtype, reserve=128 * T)
            y = ctx.ws.get("expert_rows_out", 128 * T, (self.D,), torch.float32, reserve=128 * T)
            scratch = ctx.ws.get("expert_places", ctx.ws.max_rows * self.top + T, (), torch.int32,
                                 reserve=ctx.ws.max_rows * self.top + T)
            delta = ctx.ws.get(out, N, (self.D,), ctx.dtype)
            ops.moe_tc5(h, ids, wts, self.wgu, self.wd, delta, rows, act, y, scratch, self.limit, self.alpha, self.shift, ys, gate)
            return delta, None
        y = ctx.ws.get("expert_out", N, (self.top, self.D), torch.float32)
        if ops.moe_grouped_supports(N, self.D, self.F, ctx.dtype) and not ctx.options.get("plain_experts", False):
            act = ctx.ws.get("expert_act", N * self.top, (self.F,), ctx.dtype, reserve=ctx.ws.max_rows * self.top)
            n = ops.moe_grouped_scratch(ctx.ws.max_rows, self.top, self.E)
            scratch = ctx.ws.get("expert_sort", max(n, ops.moe_grouped_scratch(N, self.top, self.E)), (), torch.int32, reserve=n)
            ops.moe_grouped(h, ids, self.wg, self.wu, self.wd, y, act, scratch, self.limit, self.alpha, self.shift)
        else:
            # bfloat16 steps of many tokens take the other form: room for the few
            most = min(ctx.ws.max_rows, max(N, ops.MOE_GROUPED["tokens"])) if ctx.dtype == torch.bfloat16 else ctx.ws.max_rows
            act = ctx.ws.get("expert_act_few", N * self.top, (self.F,), torch.float32, reserve=most * self.top)
            ops.moe_experts(h, ids, self.wg, self.wu, self.wd, y, self.limit, self.alpha, act, self.shift)
        delta = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.moe_combine(y, wts, delta, ys, gate)
        return delta, None


register("feed_forward", "routed_experts", RoutedExperts)
