"""The Fipitar decoder as data: which parts each layer has, in which order layers run and which tensors exist under which
names.

Token rows enter the stream as they are.  Every layer is a block whose sublayers read the stream itself and whose outputs
pass a layer norm (weight and bias) before they join it (`norm_after`); the model's last norm is of the same kind.  A
layer's mixer is gated linear attention (a matrix state per head and request with a decay per key channel, nothing kept
per position), latent attention (one latent vector and one rotated key strip kept per position; a sink in the softmax),
or two mixers side by side whose scaled outputs are added -- attention with normed, partly rotated heads, capped scores,
a sink of score zero and a gate per head, over cached keys and values of different widths, beside a state-space
recurrence (a matrix state per head with one decay per head and token, behind a short causal convolution).  Its
feed-forward is a dense gated unit with clamps, or absent.  A gla layer names no cache and state i; a latent layer cache
i; a side-by-side layer cache i and state i.  Stored names: `embed`, `l<i>.norm1|norm2[.b]`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down`, `final.norm[.b]`, `head`.
"""
from ..config.fipitar import FipitarConfig
from ..parts.base import LayerRun, LayerSpec, ModelSpec, PartSpec

DEFAULT_RANK = 16       # inner width of a gla layer's decay product when random weights are made and none is given
GATE_SLOPE = 1.702      # the feed-forward's gate: g sigmoid(GATE_SLOPE g)
YARN_GAIN = 0.1         # cos and sin of a scaled rotation are multiplied by YARN_GAIN ln(factor) + 1


def _rope(rot, head_dim, pairing):
    if rot is None:
        return None
    scaling = ("yarn",) + tuple(rot.scaling) + (YARN_GAIN,) if rot.scaling else None
    return PartSpec("rope", head_dim=head_dim, rotary_dim=rot.dims, theta=rot.base, pairing=pairing, scaling=scaling)


def model_spec(c: FipitarConfig) -> ModelSpec:
    D, eps = c.width, c.norm_eps
    norm = PartSpec("layer", width=D, eps=eps)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if layer.type == "gla":
            mixer = PartSpec("gla", hidden=D, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau, eps=eps, decay_rank=m.a_rank,
                             names={k: "mix." + v for k, v in dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1",
                                                                   a2="a2", a2_bias="a2.b").items()})
            run = LayerRun(layer=i, cache=None, write=False, state=i)
        elif layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", hidden=D, heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank,
                             kv_rank=m.kv_rank, eps=eps, scale=m.scale, gate=False, rot_dim=m.rot_dim,
                             position=_rope(m.rot, m.rot_dim, "adjacent"), sink="sink",
                             names={k: "mix." + v for k, v in dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv",
                                                                   dkv_norm="dkv.norm", uk="uk", uv="uv", o="o",
                                                                   sink="sink").items()})
            run = LayerRun(layer=i, cache=i, write=True)
        else:
            a, r = m.left, m.right
            left = PartSpec("gated_attention", hidden=D, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, vdim=a.vdim,
                            scale=a.scale, softcap=a.softcap, qk_norm=True, eps=eps, sink="unit", gate=True,
                            position=_rope(a.rot, a.dim, "halves"))
            right = PartSpec("ssd", hidden=D, heads=r.heads, vdim=r.vdim, state=r.state, groups=r.groups,
                             norm_groups=r.norm_groups, taps=r.conv, eps=eps)
            mixer = PartSpec("side_by_side", hidden=D, left=left, right=right, eps=eps, left_prefix="mix.left.",
                             right_prefix="mix.right.", combine="sum", left_scale=m.left_scale, right_scale=m.right_scale)
            run = LayerRun(layer=i, cache=i, write=True, state=i)
        f = layer.mlp
        ffn = None
        if f is not None:
            ffn = PartSpec("glu_clamped", hidden=D, intermediate=f.ff, limit=f.limit, alpha=GATE_SLOPE,
                           names=dict(gate="mlp.gate", up="mlp.up", down="mlp.down"))
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("norm_after", mixer=mixer, ffn=ffn, norm=norm)))
        schedule.append(run)
    return ModelSpec(hidden=D, vocab=c.vocab,
                     embedding=PartSpec("table", vocab=c.vocab, hidden=D, name="embed"),
                     layers=layers, schedule=schedule,
                     final_norm=PartSpec("layer", width=D, eps=eps, name="final.norm"),
                     head=PartSpec("linear", vocab=c.vocab, hidden=D, tied=False, name="head"))


def canonical_names(c: FipitarConfig):
    """stored names are the canonical ones; a name outside the configuration's table is unexpected"""
    known = set(stored_tensors(c))

    def canonical(name):
        if name not in known:
            raise KeyError(name)
        return name, None
    return canonical


def stored_tensors(c: FipitarConfig):
    """names, shapes and kinds of the tensors a checkpoint of this configuration holds"""
    D = c.width
    out = {"embed": ((c.vocab, D), "matrix")}

    def norm(name):
        out[name] = ((D,), "norm")
        out[name + ".b"] = ((D,), "bias")

    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        norm(p + "norm1")
        x = p + "mix."
        if layer.type == "gla":
            rank = m.a_rank or DEFAULT_RANK
            for r in "qk":
                out[x + r] = ((m.heads * m.dim, D), "matrix")
            for r in "vg":
                out[x + r] = ((m.heads * m.vdim, D), "matrix")
            out[x + "o"] = ((D, m.heads * m.vdim), "matrix")
            out[x + "norm"] = ((m.vdim,), "norm")
            out[x + "a1"] = ((rank, D), "matrix")
            out[x + "a2"] = ((m.heads * m.dim, rank), "matrix")
            out[x + "a2.b"] = ((m.heads * m.dim,), "bias")
        elif layer.type == "latent_attention":
            out[x + "dq"] = ((m.q_rank, D), "matrix")
            out[x + "dq.norm"] = ((m.q_rank,), "norm")
            out[x + "uq"] = ((m.heads * (m.dim + m.rot_dim), m.q_rank), "matrix")
            out[x + "dkv"] = ((m.kv_rank + m.rot_dim, D), "matrix")
            out[x + "dkv.norm"] = ((m.kv_rank,), "norm")
            out[x + "uk"] = ((m.heads * m.dim, m.kv_rank), "matrix")
            out[x + "uv"] = ((m.heads * m.vdim, m.kv_rank), "matrix")
            out[x + "sink"] = ((m.heads,), "bias")
            out[x + "o"] = ((D, m.heads * m.vdim), "matrix")
        else:
            a, r = m.left, m.right
            y = x + "left."
            out[y + "q"] = ((a.heads * a.dim, D), "matrix")
            out[y + "k"] = ((a.kv_heads * a.dim, D), "matrix")
            out[y + "v"] = ((a.kv_heads * a.vdim, D), "matrix")
            out[y + "q.norm"] = ((a.dim,), "norm")
            out[y + "k.norm"] = ((a.dim,), "norm")
            out[y + "g"] = ((a.heads, D), "matrix")
            out[y + "o"] = ((D, a.heads * a.vdim), "matrix")
            y = x + "right."
            inner, bc = r.heads * r.vdim, 2 * r.groups * r.state
            out[y + "in"] = ((2 * inner + bc + r.heads, D), "matrix")
            out[y + "conv"] = ((inner + bc, r.conv), "matrix")
            out[y + "conv.b"] = ((inner + bc,), "bias")
            out[y + "dt_bias"] = ((r.heads,), "bias")
            out[y + "A_log"] = ((r.heads,), "bias")
            out[y + "D"] = ((r.heads,), "norm")
            out[y + "norm"] = ((inner,), "norm")
            out[y + "o"] = ((D, inner), "matrix")
        f = layer.mlp
        if f is not None:
            norm(p + "norm2")
            out[p + "mlp.gate"] = ((f.ff, D), "matrix")
            out[p + "mlp.up"] = ((f.ff, D), "matrix")
            out[p + "mlp.down"] = ((D, f.ff), "matrix")
    norm("final.norm")
    out["head"] = ((c.vocab, D), "matrix")
    return out
