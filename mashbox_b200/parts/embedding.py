"""Token embedding (rows gathered into the float32 residual stream, src/mashbox/gguf/archs/dense.py:328-329) and the
output head (logits = h W^T in float32; the head is the embedding table when the model ties them, dense.py:129, 390)."""
from ..weights.loader import Want
from .base import make, register


class Embedding:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, vocab, hidden, name="token_embd.weight", scale=1.0):
        """scale: every row is multiplied by it on its way into the stream"""
        self.V, self.D, self.name, self.scale = int(vocab), int(hidden), name, float(scale)
        self.table = None

    def wants(self):
        return [Want(self.name, (self.V, self.D), "matrix")]

    def bind(self, tensors, env):
        self.table = tensors[self.name]

    def forward(self, ctx, x):
        ctx.ops.embed(ctx.dev("token_ids"), self.table, x, ctx.err, self.scale)


class PositionedEmbedding(Embedding):
    """x = table[token] * scale + positions[p]: a learned vector per position (counted from 0 in each sequence) is added
    to the token's row, unscaled.  The table's length bounds the context; a position beyond it is a device error."""
    graph_safe = True

    def __init__(self, vocab, hidden, max_positions, name="token_embd.weight", position_name="position_embd.weight",
                 scale=1.0):
        super().__init__(vocab, hidden, name, scale)
        self.P, self.position_name = int(max_positions), position_name
        self.context_limit = self.P         # the engine admits no request that would grow beyond the table
        self.positions = None

    def wants(self):
        return super().wants() + [Want(self.position_name, (self.P, self.D), "matrix")]

    def bind(self, tensors, env):
        super().bind(tensors, env)
        self.positions = tensors[self.position_name]

    def forward(self, ctx, x):
        ctx.ops.embed_positions(ctx.dev("token_ids"), ctx.dev("positions"), self.table, self.positions, x, ctx.err,
                                self.scale)


class NormedEmbedding(Embedding):
    """x = norm(table[token] * scale): the token's row goes through a norm of the model's kind (`norm`: its spec) on its
    way into the stream.  The norm must be one that works element by element and can write the float32 stream in place
    (`forward(..., out=)`)."""
    graph_safe = True

    def __init__(self, vocab, hidden, norm, name="token_embd.weight", scale=1.0):
        super().__init__(vocab, hidden, name, scale)
        self.norm = make("norm", norm)

    def wants(self):
        return super().wants() + self.norm.wants()

    def bind(self, tensors, env):
        super().bind(tensors, env)
        self.norm.bind(tensors, env)

    def forward(self, ctx, x):
        super().forward(ctx, x)
        self.norm.forward(ctx, x, None, out=x)


class LinearHead:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays
    def __init__(self, vocab, hidden, tied, name="output.weight", tied_to="token_embd.weight", scale=1.0):
        """scale: the logits are multiplied by it (in float32, after the product)"""
        self.V, self.D, self.tied, self.name, self.tied_to = int(vocab), int(hidden), bool(tied), name, tied_to
        self.scale = float(scale)
        self.weight = None

    def wants(self):
        return [] if self.tied else [Want(self.name, (self.V, self.D), "matrix")]

    def bind(self, tensors, env):
        self.weight = tensors[self.tied_to if self.tied else self.name]

    def forward(self, ctx, h):
        import torch
        out = ctx.ws.get("logits", h.shape[0], (self.V,), torch.float32, reserve=ctx.options.get("logit_rows", 8))
        ctx.ops.linear(h, self.weight, out=out, out_dtype=torch.float32)
        if self.scale != 1.0:
            ctx.ops.scale_rows(out, self.scale)
        return out


register("embedding", "table", Embedding)
register("embedding", "table_positions", PositionedEmbedding)
register("embedding", "table_normed", NormedEmbedding)
register("head", "linear", LinearHead)
