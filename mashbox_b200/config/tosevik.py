"""Typed configuration of the Tosevik decoder, read from config.json's own keys.

config.json: `architecture` (a string), `width`, `vocab`, `norm.eps` and `layers`, a list with one entry per layer: `type`
("retention" or "parallel"), `mixer` (its sizes and constants) and `mlp` ({"kind": "moe", "expert": {"ff"}, "router":
{"experts", "top", "scale", "groups": {"count", "keep"}}, "shared": {"ff"}} or null).  Every layer has its own sizes;
nothing is assumed equal between layers.

A retention mixer: heads, dim, vdim, decay (a number per head), rot {dims, base} (absent: no rotation).  A parallel mixer
holds two: `left`, attention with sigmoid weights (heads, kv_heads, dim, vdim, scale, q_temp {coef, every} or absent),
and `right`, a retention mixer.  Absent optional keys mean the mechanism is absent: no groups, a router scale of 1, no
shared expert, no query temperature.
"""
from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class RetentionMixer:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot_dims: int = 0                   # 0: no rotation
    rot_base: float = 10000.0


@dataclass(frozen=True)
class SigmoidMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: Optional[float] = None   # None: no query temperature
    temp_every: Optional[int] = None


@dataclass(frozen=True)
class PairMixer:
    left: SigmoidMixer
    right: RetentionMixer


@dataclass(frozen=True)
class ExpertsFF:
    ff: int
    experts: int
    top: int
    scale: float = 1.0
    groups: int = 1
    keep: int = 1
    shared_ff: Optional[int] = None     # None: no shared expert


@dataclass(frozen=True)
class TosevikLayer:
    type: str
    mixer: object
    mlp: object                         # ExpertsFF or None


@dataclass(frozen=True)
class TosevikConfig:
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
    def from_hf(cls, cfg: dict) -> "TosevikConfig":
        arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]

        def need(d, key, where):
            if not isinstance(d, dict) or d.get(key) is None:
                raise ConfigError(f"config.json has no `{where}{key}`")
            return d[key]

        def retention(m, w):
            heads = int(need(m, "heads", w))
            decay = tuple(float(d) for d in need(m, "decay", w))
            if len(decay) != heads:
                raise ConfigError(f"config.json {w}decay has {len(decay)} values for {heads} heads")
            rot, dim = m.get("rot") or {}, int(need(m, "dim", w))
            dims = int(rot.get("dims") or 0)
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json {w}rot.dims = {dims} must be even and at most dim = {dim}")
            return RetentionMixer(heads=heads, dim=dim, vdim=int(need(m, "vdim", w)), decay=decay, rot_dims=dims,
                                  rot_base=float(need(rot, "base", w + "rot.")) if dims else 10000.0)

        def sigmoid(m, w):
            heads = int(need(m, "heads", w))
            kv = int(m.get("kv_heads") or heads)
            if kv < 1 or heads % kv:
                raise ConfigError(f"config.json {w}kv_heads = {kv} does not divide heads = {heads}")
            qt = m.get("q_temp") or None
            return SigmoidMixer(heads=heads, kv_heads=kv, dim=int(need(m, "dim", w)), vdim=int(need(m, "vdim", w)),
                                scale=float(need(m, "scale", w)),
                                temp_coef=float(need(qt, "coef", w + "q_temp.")) if qt else None,
                                temp_every=int(need(qt, "every", w + "q_temp.")) if qt else None)

        layers = []
        for i, e in enumerate(need(cfg, "layers", "")):
            w = f"layers[{i}]."
            kind, m = need(e, "type", w), need(e, "mixer", w)
            w += "mixer."
            if kind == "retention":
                mixer = retention(m, w)
            elif kind == "parallel":
                mixer = PairMixer(sigmoid(need(m, "left", w), w + "left."), retention(need(m, "right", w), w + "right."))
            else:
                raise ConfigError(f"config.json layers[{i}].type = {kind!r} is not supported for {arch}")
            mlp, w = e.get("mlp"), f"layers[{i}].mlp."
            if mlp is None:
                ff = None
            elif mlp.get("kind", "moe") == "moe":
                ex, r = need(mlp, "expert", w), need(mlp, "router", w)
                groups, shared = r.get("groups") or {}, mlp.get("shared") or {}
                ff = ExpertsFF(ff=int(need(ex, "ff", w + "expert.")), experts=int(need(r, "experts", w + "router.")),
                               top=int(need(r, "top", w + "router.")), scale=float(r.get("scale", 1.0)),
                               groups=int(groups.get("count") or 1), keep=int(groups.get("keep") or groups.get("count") or 1),
                               shared_ff=int(shared["ff"]) if shared.get("ff") else None)
                if ff.experts % ff.groups or not 1 <= ff.keep <= ff.groups or not 1 <= ff.top <= ff.keep * (ff.experts // ff.groups):
                    raise ConfigError(f"config.json {w}router: {ff.top} of {ff.experts} experts in {ff.groups} groups of "
                                      f"which {ff.keep} are kept cannot be chosen")
            else:
                raise ConfigError(f"config.json {w}kind = {mlp.get('kind')!r} is not supported for {arch}")
            layers.append(TosevikLayer(kind, mixer, ff))
        return cls(architecture=arch, width=int(need(cfg, "width", "")), vocab=int(need(cfg, "vocab", "")),
                   norm_eps=float(need(cfg.get("norm"), "eps", "norm.")), layers=tuple(layers),
                   extra={k: cfg[k] for k in ("bos_token_id", "eos_token_id") if k in cfg})

    def to_hf(self) -> dict:
        """The config.json that `from_hf` reads back to this configuration (random-weights mode writes it)."""
        def retention(m):
            e = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            if m.rot_dims:
                e["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            return e

        def sigmoid(m):
            e = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.temp_coef is not None:
                e["q_temp"] = {"coef": m.temp_coef, "every": m.temp_every}
            return e

        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
               "layers": []}
        for layer in self.layers:
            m, f = layer.mixer, layer.mlp
            e = retention(m) if layer.type == "retention" else {"left": sigmoid(m.left), "right": retention(m.right)}
            mlp = None
            if f is not None:
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.scale,
                                  "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            out["layers"].append({"type": layer.type, "mixer": e, "mlp": mlp})
        out.update(self.extra)
        return out
