"""`VutesunConfig`: the config.json of a Vutesun decoder, typed and validated.

The file is nested: `layers` lists the layers in order, each with its `type` (which mixer), the mixer's sizes
under `mixer` and its feed-forward under `mlp` (null: none); `norm.eps`, `residual_mult`, `vocab` and `width`
are the model's.  Nothing is defaulted: a key the design has is required, and every error names its key.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class RotaryDims:
    base: float
    dims: int


@dataclass(frozen=True)
class SinkAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryDims


@dataclass(frozen=True)
class RetentionSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: RotaryDims


@dataclass(frozen=True)
class MLSTMSizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelSizes:
    left: SinkAttention
    right: RetentionSizes


@dataclass(frozen=True)
class ExpertsSizes:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class VutesunLayer:
    type: str                            # "mlstm" | "parallel"
    mixer: object                        # MLSTMSizes | ParallelSizes
    mlp: ExpertsSizes | None


def _rot(raw, where, head_dim) -> RotaryDims:
    r = ConfigReader(raw if raw is not None else {}, where)
    rot = RotaryDims(r.float("base", positive=True), r.int("dims", min=0))
    if rot.dims % 2 or rot.dims > head_dim:
        raise ConfigError(f"{where}: 'dims' {rot.dims} must be even and at most the head's 'dim' {head_dim}")
    return rot


def _mixer(kind: str, raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: 'mixer' must be an object")
    if kind == "mlstm":
        r = ConfigReader(raw, where)
        return MLSTMSizes(r.int("heads", min=1), r.int("dim", min=1), r.int("vdim", min=1), r.float("gate_cap", positive=True))
    if kind == "parallel":
        l = ConfigReader(raw.get("left"), f"{where}.left")
        heads, kv = l.int("heads", min=1), l.int("kv_heads", min=1)
        if heads % kv:
            raise ConfigError(f"{where}.left: 'heads' {heads} is not a multiple of 'kv_heads' {kv}")
        dim = l.int("dim", min=1)
        left = SinkAttention(heads, kv, dim, l.int("vdim", min=1), l.float("scale", positive=True),
                             _rot(l.any("rot"), f"{where}.left.rot", dim))
        r = ConfigReader(raw.get("right"), f"{where}.right")
        heads, dim = r.int("heads", min=1), r.int("dim", min=1)
        decay = r.any("decay")
        if not (isinstance(decay, list) and len(decay) == heads and all(isinstance(x, (int, float)) and not isinstance(x, bool)
                                                                        for x in decay)):
            raise ConfigError(f"{where}.right: 'decay' must list one number per head ({heads})")
        right = RetentionSizes(heads, dim, r.int("vdim", min=1), tuple(float(x) for x in decay),
                               _rot(r.any("rot"), f"{where}.right.rot", dim))
        return ParallelSizes(left, right)
    raise ConfigError(f"{where}: layer type {kind!r} is not one of 'mlstm', 'parallel'")


def _mlp(raw, where: str):
    if raw is None:
        return None
    r = ConfigReader(raw, where)
    kind = r.str("kind")
    if kind != "moe":
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is not 'moe'")
    e = ConfigReader(r.any("expert"), f"{where}.expert")
    ro = ConfigReader(r.any("router"), f"{where}.router")
    out = ExpertsSizes(e.int("ff", min=1), ro.int("experts", min=1), ro.int("top", min=1))
    if out.top > out.experts:
        raise ConfigError(f"{where}.router: 'top' {out.top} exceeds 'experts' {out.experts}")
    return out


@dataclass(frozen=True)
class VutesunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "VutesunConfig":
        r = ConfigReader(raw, where)
        layers_raw = r.any("layers")
        if not (isinstance(layers_raw, list) and layers_raw):
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            l = ConfigReader(lr, w)
            kind = l.str("type")
            layers.append(VutesunLayer(kind, _mixer(kind, l.any("mixer"), f"{w}.mixer"), _mlp(l.any("mlp"), f"{w}.mlp")))
        norm = ConfigReader(r.any("norm"), f"{where}: norm")
        return cls(architecture=r.str("architecture", "Vutesun"), vocab=r.int("vocab", min=1), width=r.int("width", min=1),
                   norm_eps=norm.float("eps", positive=True), residual_mult=r.float("residual_mult"), layers=tuple(layers))

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
        def rot(x):
            return {"base": x.base, "dims": x.dims}
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "mlstm":
                mixer = {"dim": m.dim, "gate_cap": m.gate_cap, "heads": m.heads, "vdim": m.vdim}
            else:
                a, b = m.left, m.right
                mixer = {"left": {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "rot": rot(a.rot), "scale": a.scale,
                                  "vdim": a.vdim},
                         "right": {"decay": list(b.decay), "dim": b.dim, "heads": b.heads, "rot": rot(b.rot), "vdim": b.vdim}}
            mlp = None if l.mlp is None else {"expert": {"ff": l.mlp.ff}, "kind": "moe",
                                              "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            layers.append({"mixer": mixer, "mlp": mlp, "type": l.type})
        return {"architecture": self.architecture, "layers": layers, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    def num_parameters(self) -> int:
        from ..models.registry import expected_tensors
        n = 0
        for spec in expected_tensors(self).values():
            k = 1
            for s in spec.shape:
                k *= s
            n += k
        return n
