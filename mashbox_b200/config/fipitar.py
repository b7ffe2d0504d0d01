"""Typed configuration of the Fipitar decoder, read from config.json's own keys.

config.json: `architecture` (a string), `width`, `vocab`, `norm.eps` and `layers`, a list with one entry per layer: `type`
("gla", "latent_attention" or "parallel"), `mixer` (its sizes and constants) and `mlp` ({"kind": "dense", "ff", "limit"} or
null).  Every layer has its own sizes; nothing is assumed equal between layers.

A gla mixer (gated linear attention): heads, dim, vdim, tau.  The inner width of its decay's low-rank product is not in
config.json: the stored tensors have it (`a_rank` here is None then; random-weights mode sets it and writes it as a key
of its own).  A latent_attention mixer: heads, dim (unrotated), rot_dim (rotated; absent: none), vdim, q_rank, kv_rank,
scale, rot {base, dims, scaling {factor, original, fast, slow} or absent}.  A parallel mixer holds two, `left` (attention:
heads, kv_heads, dim, vdim, scale, softcap or absent, rot {base, dims} or absent) and `right` (state-space duality: heads,
vdim, state, groups, norm_groups, conv), and the weights of their sum, `left_scale` and `right_scale`.
"""
from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[tuple] = None     # (factor, original, fast, slow) or None


@dataclass(frozen=True)
class GlaMixer:
    heads: int
    dim: int
    vdim: int
    tau: float
    a_rank: Optional[int] = None        # inner width of the decay's low-rank product; None: as stored


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dim: int = 0
    rot: Optional[Rotation] = None


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    rot: Optional[Rotation] = None


@dataclass(frozen=True)
class SsdMixer:
    heads: int
    vdim: int
    state: int
    groups: int = 1
    norm_groups: int = 1
    conv: int = 1


@dataclass(frozen=True)
class PairMixer:
    left: AttentionMixer
    right: SsdMixer
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass(frozen=True)
class DenseFF:
    ff: int
    limit: float


@dataclass(frozen=True)
class FipitarLayer:
    type: str
    mixer: object
    mlp: Optional[DenseFF]


@dataclass(frozen=True)
class FipitarConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    layers: tuple
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_hf(cls, cfg: dict) -> "FipitarConfig":
        arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]

        def need(d, key, where):
            if not isinstance(d, dict) or d.get(key) is None:
                raise ConfigError(f"config.json has no `{where}{key}`")
            return d[key]

        def rotation(m, w, most):
            rot = m.get("rot") or None
            if not rot or not rot.get("dims"):
                return None
            dims = int(rot["dims"])
            if dims % 2 or dims > most:
                raise ConfigError(f"config.json {w}rot.dims = {dims} must be even and at most {most}")
            sc = rot.get("scaling") or None
            scaling = None
            if sc:
                scaling = tuple(float(need(sc, k, w + "rot.scaling.")) for k in ("factor", "original", "fast", "slow"))
            return Rotation(dims=dims, base=float(need(rot, "base", w + "rot.")), scaling=scaling)

        def gla(m, w):
            return GlaMixer(heads=int(need(m, "heads", w)), dim=int(need(m, "dim", w)), vdim=int(need(m, "vdim", w)),
                            tau=float(need(m, "tau", w)), a_rank=int(m["a_rank"]) if m.get("a_rank") else None)

        def latent(m, w):
            rd = int(m.get("rot_dim") or 0)
            return LatentMixer(heads=int(need(m, "heads", w)), dim=int(need(m, "dim", w)), vdim=int(need(m, "vdim", w)),
                               q_rank=int(need(m, "q_rank", w)), kv_rank=int(need(m, "kv_rank", w)),
                               scale=float(need(m, "scale", w)), rot_dim=rd, rot=rotation(m, w, rd) if rd else None)

        def attention(m, w):
            heads = int(need(m, "heads", w))
            kv = int(m.get("kv_heads") or heads)
            if kv < 1 or heads % kv:
                raise ConfigError(f"config.json {w}kv_heads = {kv} does not divide heads = {heads}")
            dim = int(need(m, "dim", w))
            return AttentionMixer(heads=heads, kv_heads=kv, dim=dim, vdim=int(need(m, "vdim", w)),
                                  scale=float(need(m, "scale", w)),
                                  softcap=float(m["softcap"]) if m.get("softcap") else None, rot=rotation(m, w, dim))

        def ssd(m, w):
            heads, groups = int(need(m, "heads", w)), int(m.get("groups") or 1)
            parts, vdim = int(m.get("norm_groups") or 1), int(need(m, "vdim", w))
            if groups < 1 or heads % groups:
                raise ConfigError(f"config.json {w}groups = {groups} does not divide heads = {heads}")
            if parts < 1 or (heads * vdim) % parts:
                raise ConfigError(f"config.json {w}norm_groups = {parts} does not divide heads * vdim = {heads * vdim}")
            return SsdMixer(heads=heads, vdim=vdim, state=int(need(m, "state", w)), groups=groups, norm_groups=parts,
                            conv=int(m.get("conv") or 1))

        layers = []
        for i, e in enumerate(need(cfg, "layers", "")):
            w = f"layers[{i}]."
            kind, m = need(e, "type", w), need(e, "mixer", w)
            w += "mixer."
            if kind == "gla":
                mixer = gla(m, w)
            elif kind == "latent_attention":
                mixer = latent(m, w)
            elif kind == "parallel":
                mixer = PairMixer(attention(need(m, "left", w), w + "left."), ssd(need(m, "right", w), w + "right."),
                                  left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)))
            else:
                raise ConfigError(f"config.json layers[{i}].type = {kind!r} is not supported for {arch}")
            mlp, w = e.get("mlp"), f"layers[{i}].mlp."
            if mlp is None:
                ff = None
            elif mlp.get("kind", "dense") == "dense":
                ff = DenseFF(ff=int(need(mlp, "ff", w)), limit=float(need(mlp, "limit", w)))
            else:
                raise ConfigError(f"config.json {w}kind = {mlp.get('kind')!r} is not supported for {arch}")
            layers.append(FipitarLayer(kind, mixer, ff))
        return cls(architecture=arch, width=int(need(cfg, "width", "")), vocab=int(need(cfg, "vocab", "")),
                   norm_eps=float(need(cfg.get("norm"), "eps", "norm.")), layers=tuple(layers),
                   extra={k: cfg[k] for k in ("bos_token_id", "eos_token_id") if k in cfg})

    def to_hf(self) -> dict:
        """The config.json that `from_hf` reads back to this configuration (random-weights mode writes it)."""
        def rotation(r):
            e = {"base": r.base, "dims": r.dims}
            if r.scaling:
                e["scaling"] = dict(zip(("factor", "original", "fast", "slow"), r.scaling))
            return e

        def attention(m):
            e = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.softcap:
                e["softcap"] = m.softcap
            if m.rot:
                e["rot"] = rotation(m.rot)
            return e

        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
               "layers": []}
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "gla":
                e = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau}
                if m.a_rank:
                    e["a_rank"] = m.a_rank
            elif layer.type == "latent_attention":
                e = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                     "scale": m.scale}
                if m.rot_dim:
                    e["rot_dim"] = m.rot_dim
                if m.rot:
                    e["rot"] = rotation(m.rot)
            else:
                r = m.right
                e = {"left": attention(m.left),
                     "right": {"heads": r.heads, "vdim": r.vdim, "state": r.state, "groups": r.groups,
                               "norm_groups": r.norm_groups, "conv": r.conv},
                     "left_scale": m.left_scale, "right_scale": m.right_scale}
            mlp = None if layer.mlp is None else {"kind": "dense", "ff": layer.mlp.ff, "limit": layer.mlp.limit}
            out["layers"].append({"type": layer.type, "mixer": e, "mlp": mlp})
        out.update(self.extra)
        return out
