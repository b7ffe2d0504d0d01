"""Attention whose weights are sigmoids: every visible key counts by itself, nothing is normalised over the keys.

    q = Wq h (heads x dim), k = Wk h (kv_heads x dim), v = Wv h (kv_heads x vdim); query head h reads kv head
    h // (heads / kv_heads); no biases, no rotation
    q <- q / rms(q) * nq and k <- k / rms(k) * nk, the root mean square taken over the WHOLE row (all heads at once)
    q <- q * (1 + coef ln(floor((p + 1) / every) + 1)) at position p     (`q_temp = (coef, every)`; None: no such factor)
    v_g <- v_g / rms(v_g) per kv head, and is cached so
    weight(i, j) = sigmoid(scale q_i . k_j - slope_h (i - j) + b_h) for j <= i;   o_i = sum_j weight(i, j) v_j
    out = Wo concat_h o_h

`slopes` are one number per query head (a model hands them in; `geometric_slopes(heads, 8)` gives 2^(-8 (h+1) / heads)).
A position's cache row is a key of (kv_heads, dim) and a value of (kv_heads, vdim), both after their norms.  Norms,
scores, weights and sums are float32.

Kernels: the float32 path, and head sizes that are no multiples of 16 up to 128, use the plain kernel (a warp per token
and head, keys in ascending order).  The bfloat16 path packs the query heads of a kv head into the rows of an MMA tile:
tiles of 64 rows for prompt portions (on tcgen05, two tiles of 128 rows that share the keys, when keys and values are both
64 or both 128 wide), tiles of 16 with the keys split over warps and over blocks for decode tokens; `prepare` builds both
work lists on the host.  A weight reaches the second product as two bfloat16 numbers (hi + lo).
"""
import numpy as np

from ..cache.manager import CacheNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import register
from .diff_attention import plan_diff_attention


def geometric_slopes(heads, span=8.0):
    """-> [2^(-span (h + 1) / heads) for h in 0 .. heads - 1]"""
    return [2.0 ** (-float(span) * (h + 1) / heads) for h in range(int(heads))]


class SigmoidAttention:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, heads, kv_heads, dim, vdim, scale, eps, slopes=None, q_temp=None, head_bias=True, prefix="",
                 names=None):
        self.D, self.H, self.G, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G < 1 or self.H % self.G:
            raise ConfigError(f"{heads} heads do not divide into {kv_heads} kv heads")
        self.scale, self.eps = float(scale), float(eps)
        self.slope_values = [float(s) for s in slopes] if slopes is not None else None
        if self.slope_values is not None and len(self.slope_values) != self.H:
            raise ConfigError(f"{len(self.slope_values)} slopes for {heads} heads")
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
        if q_temp and self.q_temp[1] < 1:
            raise ConfigError("the query temperature counts positions in runs of at least one")
        self.head_bias = bool(head_bias)
        n = dict(q="q", k="k", v="v", q_norm="q.norm", k_norm="k.norm", bias="pb", o="o")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.w_in = self.wo = self.qw = self.kw = self.pb = self.slopes = None

    def wants(self):
        H, G, D = self.H, self.G, self.D
        out = [Want(self.n["q"], (H * self.dim, D), "matrix"), Want(self.n["k"], (G * self.dim, D), "matrix"),
               Want(self.n["v"], (G * self.vdim, D), "matrix"), Want(self.n["q_norm"], (H * self.dim,), "vector"),
               Want(self.n["k_norm"], (G * self.dim,), "vector"), Want(self.n["o"], (D, H * self.vdim), "matrix")]
        if self.head_bias:
            out.append(Want(self.n["bias"], (H,), "vector"))
        return out

    def bind(self, tensors, env):
        import torch
        t = lambda k: tensors[self.n[k]]
        self.w_in = torch.cat([t("q"), t("k"), t("v")], 0).contiguous()
        self.wo, self.qw, self.kw = t("o"), t("q_norm"), t("k_norm")
        self.pb = t("bias") if self.head_bias else None
        self.slopes = (torch.tensor(self.slope_values, dtype=torch.float32, device=env.device)
                       if self.slope_values is not None else None)

    def cache_need(self):
        return CacheNeed("full", ((self.G, self.dim), (self.G, self.vdim)), None)

    def state_need(self):
        return None

    def uses_mma(self, ctx):
        import torch
        return (ctx.dtype == torch.bfloat16 and ctx.ops.sigmoid_attention_mma_supports(self.dim, self.vdim)
                and not ctx.options.get("plain_attention", False))

    def uses_tc5(self, ctx):
        """prompt-form tiles go to the tcgen05 kernel when keys and values are both 64 or both 128 wide"""
        return (ctx.options.get("attention_prefill_kernel", "tc5") == "tc5"
                and ctx.ops.sigmoid_attention_tc5_supports(self.dim, self.vdim, ctx.cache.page_size))

    def plan_key(self):
        # everything the work lists depend on (the head sizes decide the kernel and its rows per tile)
        return ("sigmoid_attention", self.H // self.G, self.G, self.dim, self.vdim)

    def prepare(self, ctx):
        """host side, for the tensor-core kernels: the lists of (sequence, row tile) work items of the prompt form and
        of (sequence, split, splits, slot) items of the decode form"""
        if not self.uses_mma(ctx):
            return
        key = self.plan_key()
        if key in ctx.memo:
            return
        ops = ctx.ops
        name = "sig%d_" % len([k for k in ctx.memo if k[0] == "sigmoid_attention"])
        tc5 = self.uses_tc5(ctx)
        plan = plan_diff_attention(ctx.q_len, ctx.pos0, self.H // self.G, self.G, None,
                                   ops.sigmoid_attention_tc5_rows() if tc5 else ops.SIGMOID_MMA_ROWS,
                                   ops.SIGMOID_DECODE_ROWS, ops.SIGMOID_MAX_SPLITS,
                                   int(ctx.options.get("attention_target_blocks", 296)), ctx.options.get("attention_splits"),
                                   quads=tc5)
        for k, v in plan.items():
            ctx.inputs.add(name + k, np.asarray(v, np.int32))
        ctx.memo[key] = dict(name=name, tc5=tc5, n_pre=len(plan["pre"]) // (4 if tc5 else 2), n_dec=len(plan["dec"]) // 4,
                             n_slots=len(plan["slots"]) // 2)

    def forward(self, ctx, h, run, out="delta"):
        ops, N = ctx.ops, ctx.N
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        rows = ctx.ws.get("sigattn_in", N, (self.w_in.shape[0],), ctx.dtype)
        ops.linear(h, self.w_in, out=rows)
        group, kpool, vpool = ctx.cache.layer_cache(run.cache)
        table = group.device_table
        page, pages = ctx.cache.page_size, ctx.cache.pool_pages
        q = ctx.ws.get("sigattn_q", N, (H * dim,), ctx.dtype)
        ops.sigmoid_attention_prep(rows, self.qw, self.kw, ctx.dev("positions"), ctx.dev("tok_row"), table, q,
                                   kpool if run.write else None, vpool if run.write else None, H, G, dim, vdim, page, pages,
                                   self.eps, self.q_temp[0], self.q_temp[1], ctx.err)
        o = ctx.ws.get("sigattn_o", N, (H * vdim,), ctx.dtype)
        self.attend(ctx, q, o, table, kpool, vpool)
        y = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.linear(o, self.wo, out=y)
        return y, None

    def attend(self, ctx, q, o, table, kpool, vpool):
        ops = ctx.ops
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        page, pages = ctx.cache.page_size, ctx.cache.pool_pages
        if not self.uses_mma(ctx):
            ops.sigmoid_attention_simple(q, o, ctx.dev("positions"), ctx.dev("tok_row"), table, kpool, vpool, self.slopes,
                                         self.pb, H, G, dim, vdim, page, pages, self.scale, ctx.err)
            return
        import torch
        plan = ctx.memo[self.plan_key()]
        nm = plan["name"]
        seqs = (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("pos0"), ctx.dev("seq_row"))
        tail = (table, kpool, vpool, self.slopes, self.pb, H, G, dim, vdim, page, pages, self.scale, ctx.err)
        if plan["n_pre"]:
            prompt_form = ops.sigmoid_attention_tc5 if plan["tc5"] else ops.sigmoid_attention_mma
            prompt_form(q, o, ctx.dev(nm + "pre"), plan["n_pre"], *seqs, *tail)
        if plan["n_dec"]:
            part_o = None
            if plan["n_slots"]:
                n = plan["n_slots"] * G * ops.SIGMOID_MAX_SPLITS * ops.SIGMOID_DECODE_ROWS
                part_o = ctx.ws.get("sigattn_part_o", n, (vdim,), torch.float32, reserve=0)
            ops.sigmoid_attention_mma_decode(q, o, ctx.dev(nm + "dec"), plan["n_dec"], ctx.dev(nm + "slots"),
                                             plan["n_slots"], part_o, *seqs, *tail)


register("mixer", "sigmoid_attention", SigmoidAttention)
