"""`DekeraxConfig`: the config.json of a Dekerax decoder, typed and validated.

The file is nested: `layers` lists the distinct layers, each with its `type` (which mixer: "attention",
"latent_attention" or "delta"), the mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none;
`kind` "dense" or "moe"); `loop` (optional) names a run of layers that is executed several times with the same
weights; `norm.eps`, `vocab` and `width` are the model's.  A key the design has is required and every error
names its key; a window (`mask`) may be absent, which means all earlier keys.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int


@dataclass(frozen=True)
class WindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    rot: Rotation | None = None


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None
    rot: Rotation


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class MoESizes:
    ff: int
    experts: int
    top: int
    shared_ff: int | None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class DekeraxLayer:
    type: str
    mixer: object
    mlp: object | None


def _window(raw, where):
    if raw is None:
        return None
    return ConfigReader(raw, where).int("size", min=1)


def _rotation(raw, where, most) -> Rotation:
    if raw is None and most == 0:                        # nothing to rotate: the constants may be left out
        return Rotation(10000.0, 0)
    r = ConfigReader(raw if raw is not None else {}, where)
    rot = Rotation(r.float("base", positive=True), r.int("dims", min=0))
    if rot.dims % 2 or rot.dims > most:
        raise ConfigError(f"{where}: 'dims' {rot.dims} must be even and at most {most}")
    return rot


def _heads(r: ConfigReader):
    heads, kv = r.int("heads", min=1), r.int("kv_heads", min=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: 'heads' {heads} is not a multiple of 'kv_heads' {kv}")
    return heads, kv


def _mixer(kind: str, raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: 'mixer' must be an object")
    r = ConfigReader(raw, where)
    if kind == "attention":
        heads, kv = _heads(r)
        dim = r.int("dim", min=1)
        rot = _rotation(raw["rot"], f"{where}.rot", dim) if raw.get("rot") is not None else None
        return WindowAttentionSizes(heads, kv, dim, r.int("vdim", min=1), r.float("scale", positive=True),
                                    _window(r.any("mask"), f"{where}.mask"), rot)
    if kind == "latent_attention":
        rot_dim = r.int("rot_dim", min=0)
        return LatentAttentionSizes(r.int("heads", min=1), r.int("dim", min=1), rot_dim, r.int("vdim", min=1),
                                    r.int("q_rank", min=1), r.int("kv_rank", min=1), r.float("scale", positive=True),
                                    _window(r.any("mask"), f"{where}.mask"), _rotation(r.any("rot"), f"{where}.rot", rot_dim))
    if kind == "delta":
        heads, kv = _heads(r)
        return DeltaSizes(heads, kv, r.int("dim", min=1), r.int("vdim", min=1), r.int("conv", min=1))
    raise ConfigError(f"{where}: layer type {kind!r} is not one of 'attention', 'latent_attention', 'delta'")


def _mlp(raw, where: str):
    if raw is None:
        return None
    r = ConfigReader(raw, where)
    kind = r.str("kind")
    if kind == "dense":
        return DenseSizes(r.int("ff", min=1))
    if kind != "moe":
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is neither 'dense' nor 'moe'")
    e = ConfigReader(r.any("expert"), f"{where}.expert")
    ro = ConfigReader(r.any("router"), f"{where}.router")
    shared = r.any("shared")
    out = MoESizes(e.int("ff", min=1), ro.int("experts", min=1), ro.int("top", min=1),
                   None if shared is None else ConfigReader(shared, f"{where}.shared").int("ff", min=1))
    if out.top > out.experts:
        raise ConfigError(f"{where}.router: 'top' {out.top} exceeds 'experts' {out.experts}")
    return out


@dataclass(frozen=True)
class DekeraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    loop: Loop | None

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "DekeraxConfig":
        r = ConfigReader(raw, where)
        layers_raw = r.any("layers")
        if not (isinstance(layers_raw, list) and layers_raw):
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            l = ConfigReader(lr, w)
            kind = l.str("type")
            layers.append(DekeraxLayer(kind, _mixer(kind, l.any("mixer"), f"{w}.mixer"), _mlp(l.any("mlp"), f"{w}.mlp")))
        loop = None
        if r.any("loop") is not None:
            lp = ConfigReader(r.any("loop"), f"{where}: loop")
            loop = Loop(lp.int("start", min=0), lp.int("stop", min=0), lp.int("times", min=1))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"{where}: loop: 0 <= start <= stop <= {len(layers)} layers, got {loop.start}, {loop.stop}")
        norm = ConfigReader(r.any("norm"), f"{where}: norm")
        return cls(architecture=r.str("architecture", "Dekerax"), vocab=r.int("vocab", min=1), width=r.int("width", min=1),
                   norm_eps=norm.float("eps", positive=True), layers=tuple(layers), loop=loop)

    def run_order(self) -> list:
        """[(layer, pass)]: the layers in the order they run; `pass` is the number of the loop's pass in front of whose
        first layer the entry stands, else None."""
        L, lp = len(self.layers), self.loop
        if lp is None or lp.stop == lp.start:
            return [(i, None) for i in range(L)]
        order = [(i, None) for i in range(lp.start)]
        for p in range(lp.times):
            order += [(i, p if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, L)]

    # what every engine front end asks of a configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    eos_token_id = None
    max_position_embeddings = None

    def to_json_dict(self) -> dict:
        def mask(m, d):
            if m.window is not None:
                d["mask"] = {"size": m.window}
            return d

        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                mixer = mask(m, {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim})
                if m.rot is not None:
                    mixer["rot"] = {"base": m.rot.base, "dims": m.rot.dims}
            elif l.type == "latent_attention":
                mixer = mask(m, {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "q_rank": m.q_rank,
                                 "rot_dim": m.rot_dim, "scale": m.scale, "vdim": m.vdim})
                if m.rot_dim:
                    mixer["rot"] = {"base": m.rot.base, "dims": m.rot.dims}
            else:
                mixer = {"conv": m.conv, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "vdim": m.vdim}
            if l.mlp is None:
                mlp = None
            elif isinstance(l.mlp, DenseSizes):
                mlp = {"ff": l.mlp.ff, "kind": "dense"}
            else:
                mlp = {"expert": {"ff": l.mlp.ff}, "kind": "moe", "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
                if l.mlp.shared_ff is not None:
                    mlp["shared"] = {"ff": l.mlp.shared_ff}
            layers.append({"mixer": mixer, "mlp": mlp, "type": l.type})
        out = {"architecture": self.architecture, "layers": layers, "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    def num_parameters(self) -> int:
        from ..models.registry import expected_tensors
        n = 0
        for spec in expected_tensors(self).values():
            k = 1
            for s in spec.shape:
                k *= s
            n += k
        return n
