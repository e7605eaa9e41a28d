"""Typed configuration of the Lubavik architecture: a decoder whose config.json lists its layers
one by one.  A layer adds the normed result of a mixer, then the normed result of a feed-forward
(if it has one), then (if the model has `token_side`) a gated input made from a second token
table.  The mixer is a matrix memory with exponential gates ("mlstm"), softmax attention with a
sink per head ("attention", which may read the keys and values of an earlier layer: `kv_from`),
or chunked softmax attention beside a gated linear attention ("parallel").  The feed-forward is
dense, a mixture of experts with an always-on shared expert, or absent.  Every size and every
constant that may differ between models comes from the file:

    {"architecture": "Lubavik", "vocab": V, "width": E, "norm": {"eps": e}, "token_side": {"dim": d},
     "layers": [{"type": "mlstm", "mixer": {"heads", "dim", "vdim", "gate_cap"},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}, "kv_from": j},
                 "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts", "top", "scale"},
                         "shared": {"ff": Fs}}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {...}},
                           "right": {"heads", "dim", "vdim", "tau"}, "left_scale", "right_scale"},
                 "mlp": null}]}

`rot`, `mask`, `kv_from`, `shared` and `token_side` may be absent: the model then has no such thing.
An optional `max_positions` bounds a request's length (positions are computed, not looked up).
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, get_float, get_int, get_str

LAYER_TYPES = ("mlstm", "attention", "parallel")
DEFAULT_MAX_POSITIONS = 1 << 16


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float

    def to_dict(self):
        return {"base": self.base, "dims": self.dims}


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class SoftmaxMixer:
    """Softmax attention with grouped key/value heads: the "attention" mixer (sinks, norm over the
    whole projection, may read another layer's keys and values) and the left side of "parallel"
    (biases, per-head norm, a chunk mask)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation] = None
    chunk: Optional[int] = None
    kv_from: Optional[int] = None

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class GatedLinearSide:
    heads: int
    dim: int
    vdim: int
    tau: float

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxMixer
    right: GatedLinearSide
    left_scale: float
    right_scale: float

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class LubavikMlp:
    kind: str                         # "dense" | "moe"
    ff: int                           # dense: inner width; moe: an expert's inner width
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    shared_ff: Optional[int] = None

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff},
             "router": {"experts": self.experts, "top": self.top, "scale": self.router_scale}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class LubavikLayer:
    type: str
    mixer: object                     # MatrixMemoryMixer | SoftmaxMixer | ParallelMixer
    mlp: Optional[LubavikMlp]

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _obj(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return v


def _read_softmax(m, where, with_kv_from):
    heads, kv = get_int(m, "heads", minimum=1), get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"config.json: key 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
    dim = get_int(m, "dim", minimum=1)
    rot = None
    if m.get("rot") is not None:
        r = _obj(m, "rot", where)
        dims = get_int(r, "dims", minimum=0)
        if dims > dim or dims % 2:
            raise ConfigError(f"config.json: key 'dims' ({dims}) must be even and at most 'dim' ({dim})")
        rot = Rotation(dims, get_float(r, "base", positive=True))
    chunk = None
    if m.get("mask") is not None:
        chunk = get_int(_obj(m, "mask", where), "size", minimum=1)
    kv_from = get_int(m, "kv_from", default=None, minimum=0) if with_kv_from else None
    return SoftmaxMixer(heads, kv, dim, get_int(m, "vdim", minimum=1), get_float(m, "scale", positive=True), rot, chunk,
                        kv_from)


def _read_mixer(kind, m, where):
    if kind == "mlstm":
        return MatrixMemoryMixer(get_int(m, "heads", minimum=1), get_int(m, "dim", minimum=1),
                                 get_int(m, "vdim", minimum=1), get_float(m, "gate_cap", positive=True))
    if kind == "attention":
        return _read_softmax(m, where, True)
    r = _obj(m, "right", where)
    right = GatedLinearSide(get_int(r, "heads", minimum=1), get_int(r, "dim", minimum=1), get_int(r, "vdim", minimum=1),
                            get_float(r, "tau", positive=True))
    return ParallelMixer(_read_softmax(_obj(m, "left", where), where + ".left", False), right,
                         get_float(m, "left_scale"), get_float(m, "right_scale"))


def _read_mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be null or an object")
    kind = get_str(mlp, "kind", choices={"dense", "moe"})
    if kind == "dense":
        return LubavikMlp("dense", get_int(mlp, "ff", minimum=1))
    router = _obj(mlp, "router", where + ".mlp")
    experts, top = get_int(router, "experts", minimum=1), get_int(router, "top", minimum=1)
    if top > experts:
        raise ConfigError(f"config.json: {where}.mlp.router: {top} chosen of {experts} experts")
    shared = None
    if mlp.get("shared") is not None:
        shared = get_int(_obj(mlp, "shared", where + ".mlp"), "ff", minimum=1)
    return LubavikMlp("moe", get_int(_obj(mlp, "expert", where + ".mlp"), "ff", minimum=1), experts, top,
                      get_float(router, "scale", default=1.0), shared)


@dataclass(frozen=True)
class LubavikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LubavikLayer, ...]
    token_side_dim: Optional[int] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None
    architecture: str = "Lubavik"

    @classmethod
    def from_dict(cls, d):
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: key 'norm' must be an object with 'eps'")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = get_str(entry, "type", choices=set(LAYER_TYPES))
            try:
                mixer = _read_mixer(kind, entry["mixer"], where + ".mixer")
                mlp = _read_mlp(entry.get("mlp"), where)
            except ConfigError as e:
                raise ConfigError(f"{e} (in {where})") from None
            if kind == "attention" and mixer.kv_from is not None:
                j = mixer.kv_from
                src = layers[j].mixer if j < i and layers[j].type == "attention" else None
                if src is None or src.kv_from is not None:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from = {j} must name an earlier attention "
                                      "layer with keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim, src.rot) != (mixer.kv_heads, mixer.dim, mixer.vdim, mixer.rot):
                    raise ConfigError(f"config.json: {where} reads the keys and values of layer {j}, whose key/value "
                                      "heads, sizes or rotation differ")
            layers.append(LubavikLayer(kind, mixer, mlp))
        side = None
        if d.get("token_side") is not None:
            side = get_int(_obj(d, "token_side", "config"), "dim", minimum=1)
        return cls(vocab=get_int(d, "vocab", minimum=1), width=get_int(d, "width", minimum=1),
                   norm_eps=get_float(norm, "eps", positive=True), layers=tuple(layers), token_side_dim=side,
                   max_positions=get_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
                   eos_token_id=get_int(d, "eos_token_id", default=None))

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.token_side_dim is not None:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
