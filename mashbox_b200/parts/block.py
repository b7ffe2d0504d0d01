"""Block arrangements: how a layer's norm, mixer and feed-forward are put together.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)) (src/mashbox/gguf/archs/dense.py:339-357).  The adds are deferred: a
sublayer returns its output as `pending` and the next norm adds it into the float32 residual stream in the same kernel
that normalises, so the block returns the feed-forward's output still pending.

"prenorm_depth": "prenorm", after which the stream is replaced by a weighted sum of everything it has been so far (see
DepthAveragedBlock).

"sandwich": a norm before AND after each sublayer, the normed output scaled per channel before it joins the stream,
and optionally an input from the token itself at the layer's end (see SandwichBlock).

"norm_after": the sublayers read the stream as it is and only their outputs are normed (see OutputNormBlock).
"""
from ..errors import ConfigError
from .base import make, register


class PreNormBlock:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, prefix, mixer, ffn, norm=None, norm1=None, norm2=None):
        """mixer, ffn: part specs; norm: the spec of both norms, or norm1 / norm2 when they differ"""
        p = prefix
        self.norm1 = make("norm", norm1 or norm, name=p + "attn_norm.weight")
        self.mixer = make("mixer", mixer, prefix=p)
        self.norm2 = make("norm", norm2 or norm, name=p + "ffn_norm.weight")
        self.ffn = make("feed_forward", ffn, prefix=p)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, ctx, x, pending, run):
        # A step of very few tokens is a chain of short kernels.  Parts that say `fuses_small` take two of them in:
        # with normed=(x, norm) their first product is the product of the normalised stream without a norm kernel (x
        # must be up to date: nothing pending; the streaming products also need what the product before left for this
        # norm, ctx.held_for), with residual=x their last product adds into the stream (ctx.add_into_stream) and
        # nothing is left pending.
        small = ctx.ops.small_fused_supports(ctx.N, x.shape[1], ctx.dtype) and not ctx.options.get("no_small_fusion", False)
        pending = self._sublayer(ctx, x, pending, self.norm1, self.mixer, small, self.norm2, run)
        return self._sublayer(ctx, x, pending, self.norm2, self.ffn, small, ctx.next_first_norm)

    def first_norm(self):
        """the norm that reads the residual stream first when this block runs"""
        return self.norm1

    @staticmethod
    def _sublayer(ctx, x, pending, norm, part, small, after, *run):
        ctx.after_norm = after                  # the norm that reads x after this part (None: not known)
        if not (small and getattr(part, "fuses_small", False) and hasattr(norm, "fusable")):
            return part.forward(ctx, norm.forward(ctx, x, pending), *run)
        ready = pending is None and (not ctx.ops.small_normed_needs_held(ctx.N, x.shape[1]) or ctx.held_for(x, norm) is not None)
        if not ready:
            return part.forward(ctx, norm.forward(ctx, x, pending), *run, residual=x)
        return part.forward(ctx, None, *run, normed=(x, norm), residual=x)


register("block", "prenorm", PreNormBlock)


class DepthAveragedBlock:
    """y = x + mixer(norm1(x));  y += ffn(norm2(y));  X_(index+1) = y;  x = sum_(j <= index+1) c[j] X_j.

    X_0 is the stream as the embedding left it and X_(j+1) the result of the block with `index` j, before this sum; the
    block with index i reads i + 2 coefficients from the tensor `coef` under its prefix.  The history is one workspace
    buffer (`total` + 1 slots of the step's rows, float32).  One kernel adds the feed-forward's output, writes the
    history slot, sums, writes the stream and -- when the norm that reads the stream next works element by element
    (`elementwise()`) -- makes that norm's output too.  `ffn` may be None.  Nothing is left pending."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, prefix, mixer, norm, index, total, ffn=None, coef="dwa", names=None):
        n = dict(norm1="norm1", norm2="norm2")
        n.update(names or {})
        self.index, self.total = int(index), int(total)
        if not 0 <= self.index < self.total:
            raise ConfigError(f"a depth-averaged block with index {index} of {total}")
        self.norm1 = make("norm", norm, name=prefix + n["norm1"])
        self.mixer = make("mixer", mixer, prefix=prefix)
        self.ffn = make("feed_forward", ffn, prefix=prefix) if ffn is not None else None
        self.norm2 = make("norm", norm, name=prefix + n["norm2"]) if self.ffn is not None else None
        self.coef_name = prefix + coef
        self.width = self.norm1.width
        self.coef = None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self) if p is not None]

    # the block is a part of its own for the coefficients
    def wants(self):
        from ..weights.loader import Want
        return [Want(self.coef_name, (self.index + 2,), "vector")]

    def bind(self, tensors, env):
        self.coef = tensors[self.coef_name]

    def first_norm(self):
        return self.norm1

    def state_need(self):
        return self.mixer.state_need()

    def prepare(self, ctx):
        self.mixer.prepare(ctx)

    def forward(self, ctx, x, pending, run):
        import torch
        ctx.after_norm = None
        hist = ctx.ws.get("depth_history", self.total + 1, (ctx.ws.max_rows, self.width), torch.float32,
                          reserve=self.total + 1)
        ready = ctx.memo.pop("prenormed", None)
        if pending is None and ready is not None and ready[0] is self.norm1 and ready[1] == x.data_ptr():
            h = ready[2]                    # the block before made this norm while it wrote the stream
        else:
            h = self.norm1.forward(ctx, x, pending)
        if self.index == 0:
            hist[0, :x.shape[0]].copy_(x)   # the stream as the embedding left it (what was pending is in by now)
        pending = self.mixer.forward(ctx, h, run)
        if self.ffn is not None:
            pending = self.ffn.forward(ctx, self.norm2.forward(ctx, x, pending))
        delta, bias = pending
        if bias is not None:
            raise ConfigError("a depth-averaged block cannot defer a bias")
        nxt = ctx.next_first_norm
        if not (nxt is not None and hasattr(nxt, "elementwise") and nxt.width == self.width):
            nxt = None
        normed = ctx.ws.get("normed", x.shape[0], (self.width,), ctx.dtype) if nxt is not None else None
        ctx.ops.depth_average(x, delta, hist, self.coef, self.index, normed, nxt.elementwise() if nxt is not None else None)
        if nxt is not None:
            ctx.memo["prenormed"] = (nxt, x.data_ptr(), normed)
        return None


register("block", "prenorm_depth", DepthAveragedBlock)


class ParallelBlock:
    """x += mixer(conv(norm1(x))) + ffn(norm2(x)): both sublayers read the same stream, each through a norm of its own.

    `mixer_conv` (optional): a short causal convolution on what the mixer reads.  `ffn` may be None.  The two outputs
    stay pending (delta of the mixer, None, delta of the feed-forward) and the next norm kernel adds both into the
    float32 stream; when the two norms are of one kind, width and eps, one kernel makes both from one sum of squares.
    The layer's state (what its convolutions carry across steps) is one flat float32 tensor per request: the input
    convolution's stretch first, then the mixer's."""

    def __init__(self, prefix, mixer, norm1, norm2=None, ffn=None, mixer_conv=None, names=None):
        n = dict(norm1="norm1", norm2="norm2", conv="canon1")
        n.update(names or {})
        self.norm1 = make("norm", norm1, name=prefix + n["norm1"])
        self.conv = make("conv", mixer_conv, name=prefix + n["conv"]) if mixer_conv is not None else None
        self.mixer = make("mixer", mixer, prefix=prefix)
        self.ffn = make("feed_forward", ffn, prefix=prefix) if ffn is not None else None
        self.norm2 = make("norm", norm2 or norm1, name=prefix + n["norm2"]) if self.ffn is not None else None
        off = 0
        for part in (self.conv, self.mixer):
            if part is not None and hasattr(part, "state_floats"):
                part.state_offset = off
                off += part.state_floats()
        self.state_total = off

    @property
    def graph_safe(self):
        return True         # forward() depends on the batch only through the lengths of the step's arrays

    def parts(self):
        return [p for p in (self.norm1, self.conv, self.mixer, self.norm2, self.ffn) if p is not None]

    def first_norm(self):
        return self.norm1

    def state_need(self):
        from ..cache.manager import StateNeed
        if hasattr(self.mixer, "state_floats"):
            return StateNeed((self.state_total,), "float32") if self.state_total else None
        if self.conv is not None and self.conv.state_floats():
            raise ConfigError("a parallel block with an input convolution needs a mixer that says how much state it keeps")
        return self.mixer.state_need()

    def prepare(self, ctx):
        for part in (self.conv, self.mixer):
            if part is not None:
                part.prepare(ctx)

    def forward(self, ctx, x, pending, run):
        ctx.after_norm = None
        conv_done = False
        if self.ffn is not None and hasattr(self.norm1, "forward_pair") and type(self.norm2) is type(self.norm1) \
                and (self.norm1.width, self.norm1.eps) == (self.norm2.width, self.norm2.eps):
            # a step in which every sequence brings one token (N == S follows from the lengths of the step's arrays): the
            # input convolution is the same kernel's work
            fold = (self.conv is not None and ctx.N == ctx.S and hasattr(self.conv, "foldable")
                    and self.conv.foldable(ctx, run.state_id) and not ctx.options.get("no_small_fusion", False))
            a, b = self.norm1.forward_pair(ctx, x, self.norm2, pending,
                                           conv=self.conv.folded(ctx, run.state_id) if fold else None)
            if fold:
                conv_done = True
        else:
            a = self.norm1.forward(ctx, x, pending)
            b = self.norm2.forward(ctx, x, None) if self.ffn is not None else None
        if self.conv is not None and not conv_done:
            a = self.conv.forward(ctx, a, run.state_id)
        delta, bias = self.mixer.forward(ctx, a, run)
        if self.ffn is None:
            return delta, bias
        if bias is not None:
            raise ConfigError("a parallel block cannot defer a bias of its mixer's output")
        side, _ = self.ffn.forward(ctx, b, out="delta_side")
        return delta, None, side


register("block", "parallel", ParallelBlock)


class SandwichBlock:
    """x += l1 * post1(mixer(pre1(x)));  x += l2 * post2(ffn(pre2(x)));  then, optionally, side(x, token) adds into x.

    pre and post norms are RMS norms; l1, l2 (`scale1`, `scale2`: tensor names under the layer's prefix, or None) scale
    the normed outputs channel by channel and are multiplied into the post norms' weights at load.  One kernel norms a
    sublayer's output, adds it into the float32 stream and makes the norm that reads the stream next -- the
    feed-forward's pre norm, or the first norm of the block that runs next -- so the stream is read once per sublayer.
    `ffn` may be None (the layer has no feed-forward), `side` may be None.  Nothing is left pending."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, prefix, mixer, norm, ffn=None, side=None, scale1=None, scale2=None, names=None):
        n = dict(pre1="norm1", post1="norm1b", pre2="norm2", post2="norm2b")
        n.update(names or {})
        self.pre1 = make("norm", norm, name=prefix + n["pre1"])
        self.post1 = make("norm", norm, name=prefix + n["post1"])
        self.mixer = make("mixer", mixer, prefix=prefix)
        self.ffn = make("feed_forward", ffn, prefix=prefix) if ffn is not None else None
        self.pre2 = make("norm", norm, name=prefix + n["pre2"]) if self.ffn is not None else None
        self.post2 = make("norm", norm, name=prefix + n["post2"]) if self.ffn is not None else None
        self.side = make("side", side, prefix=prefix) if side is not None else None
        self.scale_names = (prefix + scale1 if scale1 else None, prefix + scale2 if scale2 and self.ffn is not None else None)
        self.width = self.pre1.width
        self.post_w = [None, None]

    def parts(self):
        return [p for p in (self.pre1, self.mixer, self.post1, self.pre2, self.ffn, self.post2, self.side, self)
                if p is not None]

    # the block is a part of its own for the two scale vectors
    def wants(self):
        from ..weights.loader import Want
        return [Want(n, (self.width,), "vector") for n in self.scale_names if n is not None]

    def bind(self, tensors, env):
        for i, (post, name) in enumerate(zip((self.post1, self.post2), self.scale_names)):
            if post is not None:
                self.post_w[i] = post.weight * tensors[name] if name is not None else post.weight

    def first_norm(self):
        return self.pre1

    def state_need(self):
        return self.mixer.state_need()

    def prepare(self, ctx):
        self.mixer.prepare(ctx)

    def forward(self, ctx, x, pending, run):
        import torch
        ops = ctx.ops
        ctx.after_norm = None
        ready = ctx.memo.pop("prenormed", None)
        if pending is None and ready is not None and ready[0] is self.pre1 and ready[1] == x.data_ptr():
            h = ready[2]                    # the block before made this norm while it added its last output
        else:
            h = self.pre1.forward(ctx, x, pending)
        nxt = ctx.next_first_norm
        if not (nxt is not None and type(nxt) is type(self.pre1) and nxt.width == self.width):
            nxt = None
        steps = [(self.mixer, self.post1, self.post_w[0], (run,))]
        if self.ffn is not None:
            steps.append((self.ffn, self.post2, self.post_w[1], ()))
        xa = None
        for i, (part, post, w, args) in enumerate(steps):
            y, bias = part.forward(ctx, h, *args)
            if bias is not None:
                raise ConfigError("a sandwich block cannot norm an output with a deferred bias")
            last = i == len(steps) - 1
            follow = (self.pre2 if not last else (nxt if self.side is None else None))
            h = ctx.ws.get("normed", x.shape[0], (self.width,), ctx.dtype) if follow is not None else None
            if last and self.side is not None and ctx.dtype != torch.float32:
                xa = ctx.ws.get("stream_copy", x.shape[0], (self.width,), ctx.dtype)
            ops.post_norm_add(x, y, w, post.eps, follow.weight if follow is not None else None,
                              follow.eps if follow is not None else 0.0, h, xa)
        if self.side is not None:
            h = ctx.ws.get("normed", x.shape[0], (self.width,), ctx.dtype) if nxt is not None else None
            self.side.forward(ctx, x, x if xa is None else xa, nxt, h)
        if nxt is not None:
            ctx.memo["prenormed"] = (nxt, x.data_ptr(), h)
        return None


register("block", "sandwich", SandwichBlock)


class OutputNormBlock:
    """x += norm1(mixer(x));  x += norm2(ffn(x)): the sublayers read the stream itself, and what they return passes a
    norm before it joins the stream.

    The norm is any registered kind that offers `add_output` (norm, add into the float32 stream and the new stream in
    the activation dtype, one kernel).  A mixer that is a weighted sum of two (`forward_parts`) hands both outputs and
    their weights to that kernel instead of adding them itself.  `ffn` may be None.  Nothing is left pending; what the
    block before left pending is added first."""
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, prefix, mixer, norm, ffn=None, names=None):
        n = dict(norm1="norm1", norm2="norm2")
        n.update(names or {})
        self.norm1 = make("norm", norm, name=prefix + n["norm1"])
        self.mixer = make("mixer", mixer, prefix=prefix)
        self.ffn = make("feed_forward", ffn, prefix=prefix) if ffn is not None else None
        self.norm2 = make("norm", norm, name=prefix + n["norm2"]) if self.ffn is not None else None
        if not hasattr(self.norm1, "add_output"):
            raise ConfigError("a block that norms its sublayers' outputs needs a norm kind with add_output")
        self.width = self.norm1.width

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def state_need(self):
        return self.mixer.state_need()

    def prepare(self, ctx):
        self.mixer.prepare(ctx)

    def _stream(self, ctx, x, pending):
        """-> the stream in the activation dtype (the float32 stream itself when that is the activation dtype)"""
        import torch
        if pending is not None:
            delta, bias, *more = pending
            ctx.memo.pop("held", None)
            ctx.memo.pop("stream_rows", None)
            for d in (delta, bias, *more):
                if d is not None:
                    x.add_(d)
        if ctx.dtype == torch.float32:
            return x, None
        xa = ctx.ws.get("stream_rows", x.shape[0], (self.width,), ctx.dtype)
        ready = ctx.memo.get("stream_rows")
        if ready != x.data_ptr():
            ctx.ops.to_rows(x, xa)
            ctx.memo["stream_rows"] = x.data_ptr()
        return xa, xa

    def forward(self, ctx, x, pending, run):
        ctx.after_norm = None
        h, copy = self._stream(ctx, x, pending)
        if hasattr(self.mixer, "forward_parts"):
            a, sa, b, sb = self.mixer.forward_parts(ctx, h, run)
            self.norm1.add_output(ctx, x, a, copy, b, sa, sb)
        else:
            y, bias = self.mixer.forward(ctx, h, run)
            if bias is not None:
                raise ConfigError("a block that norms its sublayers' outputs cannot defer a bias")
            self.norm1.add_output(ctx, x, y, copy)
        if self.ffn is not None:
            y, bias = self.ffn.forward(ctx, h)
            if bias is not None:
                raise ConfigError("a block that norms its sublayers' outputs cannot defer a bias")
            self.norm2.add_output(ctx, x, y, copy)
        return None


register("block", "norm_after", OutputNormBlock)
