"""The Tosevik decoder as data: which parts each layer has, in which order layers run and which tensors exist under which
names.

Token rows go through a Dynamic Tanh norm into the stream.  Every layer is a pre-norm block with Dynamic Tanh norms
whose result is replaced, for whoever reads the stream next, by a weighted sum of the embedding's output and every
layer's result so far (`prenorm_depth`).  A layer's mixer is retention (a matrix state per head and request, nothing
kept per position) or two mixers side by side -- attention with sigmoid weights over cached keys and values, and
retention -- whose normed outputs are averaged; its feed-forward is routed experts with softmax scores, groups worth
their best expert, scaled weights and a gated shared expert, or absent.  A retention layer names no cache and a state of
its own; a side-by-side layer names cache i and state i.  Stored names: `embed`, `embed.norm[.b|.alpha]`,
`l<i>.norm1|norm2[.b|.alpha]`, `l<i>.mix.*`, `l<i>.mlp.router|e<j>.gate|up|down|shared.gate|up|down|sg`, `l<i>.dwa`,
`final.norm[.b|.alpha]`, `head`.
"""
from ..config.tosevik import TosevikConfig
from ..parts.base import LayerRun, LayerSpec, ModelSpec, PartSpec
from ..parts.sigmoid_attention import geometric_slopes

SLOPE_SPAN = 8.0        # the distance bias of head h of H: slope 2^(-SLOPE_SPAN (h + 1) / H)


def _retention(D, m, eps):
    position = PartSpec("rope", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base, pairing="halves") if m.rot_dims else None
    return PartSpec("retention", hidden=D, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), eps=eps,
                    position=position)


def _sigmoid(D, m, eps):
    return PartSpec("sigmoid_attention", hidden=D, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
                    eps=eps, slopes=geometric_slopes(m.heads, SLOPE_SPAN),
                    q_temp=[m.temp_coef, m.temp_every] if m.temp_coef is not None else None)


def model_spec(c: TosevikConfig) -> ModelSpec:
    D, eps = c.width, c.norm_eps
    norm = PartSpec("dyt", width=D, eps=eps)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if layer.type == "retention":
            mixer = PartSpec("retention", **{**_retention(D, m, eps).params, "names": {k: "mix." + k for k in "qkvgo"}})
            run = LayerRun(layer=i, cache=None, write=False, state=i)
        else:
            mixer = PartSpec("side_by_side", hidden=D, left=_sigmoid(D, m.left, eps), right=_retention(D, m.right, eps), eps=eps,
                             left_prefix="mix.left.", right_prefix="mix.right.", left_weight="mix.left.out",
                             right_weight="mix.right.out")
            run = LayerRun(layer=i, cache=i, write=True, state=i)
        f = layer.mlp
        ffn = None
        if f is not None:
            shared = None
            if f.shared_ff:
                shared = PartSpec("swiglu", hidden=D, intermediate=f.shared_ff, names=dict(gate="gate", up="up", down="down"))
            ffn = PartSpec("routed_experts", hidden=D, intermediate=f.ff, experts=f.experts, top=f.top, limit=None, alpha=1.0,
                           shift=0.0, correction=False, score="softmax", group_worth="max", scale=f.scale, groups=f.groups,
                           keep=f.keep, shared=shared, shared_prefix="mlp.shared.", shared_gate="mlp.shared.sg" if shared else None)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm_depth", mixer=mixer, ffn=ffn, norm=norm, index=i,
                                                                 total=c.num_layers, coef="dwa")))
        schedule.append(run)
    return ModelSpec(hidden=D, vocab=c.vocab,
                     embedding=PartSpec("table_normed", vocab=c.vocab, hidden=D, name="embed",
                                        norm=PartSpec("dyt", width=D, eps=eps, name="embed.norm")),
                     layers=layers, schedule=schedule,
                     final_norm=PartSpec("dyt", width=D, eps=eps, name="final.norm"),
                     head=PartSpec("linear", vocab=c.vocab, hidden=D, tied=False, name="head"))


def canonical_names(c: TosevikConfig):
    """stored names are the canonical ones, except that the shared expert's matrices get the `.weight` its part appends;
    a name outside the configuration's table is unexpected"""
    known = set(stored_tensors(c))
    dense = {f"l{i}.mlp.shared.{r}" for i, layer in enumerate(c.layers) if layer.mlp is not None and layer.mlp.shared_ff
             for r in ("gate", "up", "down")}

    def canonical(name):
        if name not in known:
            raise KeyError(name)
        return (name + ".weight" if name in dense else name), None
    return canonical


def stored_tensors(c: TosevikConfig):
    """names, shapes and kinds of the tensors a checkpoint of this configuration holds"""
    D = c.width
    out = {"embed": ((c.vocab, D), "matrix")}

    def norm(name):
        out[name] = ((D,), "norm")
        out[name + ".b"] = ((D,), "bias")
        out[name + ".alpha"] = ((), "alpha")

    def retention(x, m):
        out[x + "q"] = ((m.heads * m.dim, D), "matrix")
        out[x + "k"] = ((m.heads * m.dim, D), "matrix")
        out[x + "v"] = ((m.heads * m.vdim, D), "matrix")
        out[x + "g"] = ((m.heads * m.vdim, D), "matrix")
        out[x + "o"] = ((D, m.heads * m.vdim), "matrix")

    norm("embed.norm")
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        norm(p + "norm1")
        if layer.type == "retention":
            retention(p + "mix.", m)
        else:
            x, a = p + "mix.left.", m.left
            out[x + "q"] = ((a.heads * a.dim, D), "matrix")
            out[x + "k"] = ((a.kv_heads * a.dim, D), "matrix")
            out[x + "v"] = ((a.kv_heads * a.vdim, D), "matrix")
            out[x + "q.norm"] = ((a.heads * a.dim,), "norm")
            out[x + "k.norm"] = ((a.kv_heads * a.dim,), "norm")
            out[x + "pb"] = ((a.heads,), "bias")
            out[x + "o"] = ((D, a.heads * a.vdim), "matrix")
            retention(p + "mix.right.", m.right)
            out[p + "mix.left.out"] = ((D,), "norm")
            out[p + "mix.right.out"] = ((D,), "norm")
        f = layer.mlp
        if f is not None:
            norm(p + "norm2")
            for e in range(f.experts):
                out[f"{p}mlp.e{e}.gate"] = ((f.ff, D), "matrix")
                out[f"{p}mlp.e{e}.up"] = ((f.ff, D), "matrix")
                out[f"{p}mlp.e{e}.down"] = ((D, f.ff), "matrix")
            out[p + "mlp.router"] = ((f.experts, D), "matrix")
            if f.shared_ff:
                out[p + "mlp.shared.gate"] = ((f.shared_ff, D), "matrix")
                out[p + "mlp.shared.up"] = ((f.shared_ff, D), "matrix")
                out[p + "mlp.shared.down"] = ((D, f.shared_ff), "matrix")
                out[p + "mlp.shared.sg"] = ((1, D), "matrix")
        out[p + "dwa"] = ((i + 2,), "depth")
    norm("final.norm")
    out["head"] = ((c.vocab, D), "matrix")
    return out
