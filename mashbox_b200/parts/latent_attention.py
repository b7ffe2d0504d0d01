"""The latent attention mixer: keys and values are projections of ONE latent vector per position, and only that vector
is kept.

    cq = rms(Wdq h) nq;   q = Wuq cq  (heads x dim)
    c  = rms(Wdkv h) nkv  (kv_rank values: the row a position keeps in its page)
    k_h = Wuk_h c,  v_h = Wuv_h c;   o_h = softmax(scale q_h K_h^T) V_h over the positions up to the query's own
    out = Wo (concat_h o_h * sigmoid(Wg h))

Optional, each a constructor parameter: a rotated part (`rot_dim` > 0 with a `position` spec) -- every query head then
has dim unrotated and rot_dim rotated values, [u_h | r_h], Wdkv makes kv_rank + rot_dim rows of which the last rot_dim
(not normed) are ONE rotated key strip kr shared by all heads, the score is scale (u_h . Wuk_h c + r_h . kr), and a
position keeps [c | kr]; a sink per head (`sink`: the name of a tensor with one number per head that joins the
softmax's denominator without a value); the output gate (`gate`).

Since k_h is linear in c, the score q_h . (Wuk_h c) equals (Wuk_h^T q_h) . c, and the
weighted sum of the v_h is Wuv_h applied to the weighted sum of the c: every head attends to the SAME rows -- the
latents in their pages -- with a query of kv_rank values, and its result is brought to vdim values afterwards.  That
is attention with one kv head of head size kv_rank in which a position's row is key and value at once (with a rotated
part: keys of kv_rank + rot_dim values, [Wuk_h^T u_h | r_h] against [c | kr], values the row's first kv_rank), so the step
runs the engine's paged attention kernels (`PagedAttention`: plain, mma.sync, TMA, tcgen05 by head size) on the latent
pool, between two per-head products.  Nothing but c is ever read from the cache, whole prompts, portions and single
tokens alike.  `shares_kv`: the layer has no Wdkv and reads the latents another layer wrote (its schedule entry names
that cache), with its own Wuk, Wuv and queries.  Norms, scores, softmax and the weighted sums are float32.
"""
from ..cache.manager import CacheNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .attention import PagedAttention
from .base import PartSpec, make, register


class LatentAttention:
    @property
    def graph_safe(self):
        """forward() depends on the batch only through the lengths of the step's arrays; so must the position encoding"""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden, heads, dim, vdim, q_rank, kv_rank, eps, scale=None, gate=True, shares_kv=False, prefix="",
                 names=None, rot_dim=0, position=None, sink=None):
        self.D, self.H, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale else self.dim ** -0.5
        self.gate, self.shares_kv = bool(gate), bool(shares_kv)
        n = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o",
                 sink="sink")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.rot_dim = int(rot_dim or 0)
        self.position = make("position", position) if isinstance(position, PartSpec) else position
        self.has_sink = sink is not None
        self.row = self.kv_rank + self.rot_dim          # what a position keeps
        # every head's query of kv_rank (+ rot_dim) values over the one row a position keeps
        if self.rot_dim or self.has_sink:
            self.core = PagedAttention(self.H, 1, self.row, None, self.scale, vdim=self.kv_rank, sinks=self.has_sink)
            self.core.general = True
        else:
            self.core = PagedAttention(self.H, 1, self.kv_rank, None, self.scale)
        self.w_in = self.nq = self.nkv = self.wuq = self.wuk = self.wuv = self.wo = self.sinks = None

    def wants(self):
        H, D = self.H, self.D
        out = [Want(self.n["dq"], (self.q_rank, D), "matrix"), Want(self.n["dq_norm"], (self.q_rank,), "vector"),
               Want(self.n["uq"], (H * (self.dim + self.rot_dim), self.q_rank), "matrix"),
               Want(self.n["uk"], (H * self.dim, self.kv_rank), "matrix"),
               Want(self.n["uv"], (H * self.vdim, self.kv_rank), "matrix"),
               Want(self.n["o"], (D, H * self.vdim), "matrix")]
        if not self.shares_kv:
            out += [Want(self.n["dkv"], (self.row, D), "matrix"), Want(self.n["dkv_norm"], (self.kv_rank,), "vector")]
        if self.gate:
            out.append(Want(self.n["g"], (H * self.vdim, D), "matrix"))
        if self.has_sink:
            out.append(Want(self.n["sink"], (H,), "vector"))
        return out + (self.position.wants() if self.position is not None else [])

    def bind(self, tensors, env):
        import torch
        t = lambda k: tensors[self.n[k]]
        first = [t("dq")] + ([] if self.shares_kv else [t("dkv")]) + ([t("g")] if self.gate else [])
        self.w_in = torch.cat(first, 0).contiguous()           # one product: [query latent | kept latent | gate]
        self.nq = t("dq_norm")
        self.nkv = None if self.shares_kv else t("dkv_norm")
        self.wuq, self.wuk, self.wuv, self.wo = t("uq"), t("uk"), t("uv"), t("o")
        self.sinks = t("sink") if self.has_sink else None
        if self.position is not None:
            self.position.bind(tensors, env)
            if self.position.rotation() is None or self.position.rotation()[1] > self.rot_dim:
                raise ConfigError("latent attention rotates a strip of rot_dim values in its own kernel; its position "
                                  "part must hand it frequencies for at most that many")
        if self.rot_dim and self.shares_kv:
            raise ConfigError("a latent attention layer with a rotated part keeps its own rows")

    def cache_need(self):
        return CacheNeed("full", ((1, self.row),))

    def state_need(self):
        return None

    def prepare(self, ctx):
        self.core.prepare(ctx)

    def forward(self, ctx, h, run):
        ops, N, H = ctx.ops, ctx.N, self.H
        if run.write == self.shares_kv:
            raise ConfigError("a latent attention layer writes the cache it owns and only reads one it borrows")
        own = not self.shares_kv
        rows = ctx.ws.get("latent_in", N, (self.w_in.shape[0],), ctx.dtype)
        ops.linear(h, self.w_in, out=rows)
        group, pool = ctx.cache.layer_cache(run.cache)
        table, page, pages = group.device_table, ctx.cache.page_size, ctx.cache.pool_pages
        cq = ctx.ws.get("latent_q", N, (self.q_rank,), ctx.dtype)
        segments = ops.rms_segments_wide if self.row != self.kv_rank else ops.rms_segments
        segments(rows, 0, self.nq, cq, self.q_rank, self.nkv, pool if own else None, ctx.dev("positions"),
                 ctx.dev("tok_row"), table, page, pages, self.eps, ctx.err)
        q = ctx.ws.get("latent_heads_q", N, (H * (self.dim + self.rot_dim),), ctx.dtype)
        ops.linear(cq, self.wuq, out=q)
        qa = ctx.ws.get("latent_query", N, (H * self.row,), ctx.dtype)
        if self.rot_dim:
            ops.head_product_strided(q, self.dim, self.wuk, qa, self.kv_rank, H, transposed=True)   # Wuk_h^T u_h
            freqs, rd, pairing, gain = None, 0, 0, 1.0
            if self.position is not None:
                freqs, rd, pairing = self.position.rotation()
                gain = getattr(self.position, "gain", 1.0)
            # r_h behind it, and the token's key strip behind its latent in the page, both rotated
            ops.latent_rope(q, self.dim + self.rot_dim, self.dim, qa, self.row, self.kv_rank, rows,
                            self.q_rank + self.kv_rank, pool if own else None, self.kv_rank, freqs, rd, self.rot_dim, pairing,
                            gain, ctx.dev("positions"), ctx.dev("tok_row"), table, H, page, pages, ctx.err)
        else:
            ops.head_product(q, self.wuk, qa, H, transposed=True)               # Wuk_h^T q_h
        oa = ctx.ws.get("latent_mix", N, (H * self.kv_rank,), ctx.dtype)
        self.core.attend(ctx, qa, H * self.row, oa, table, pool, pool, sinks=self.sinks)
        o = ctx.ws.get("attn_out", N, (H * self.vdim,), ctx.dtype)
        ops.head_product(oa, self.wuv, o, H, transposed=False)                  # Wuv_h (sum of weighted latents)
        if self.gate:
            off = self.q_rank + (self.row if own else 0)
            ops.sigmoid_mul(o, rows[:, off:off + H * self.vdim])
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(o, self.wo, out=y)
        return y, None


register("mixer", "latent_attention", LatentAttention)
