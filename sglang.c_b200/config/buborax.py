"""Typed configuration of the Buborax architecture: a decoder whose config.json lists its layers
one by one.  A layer is pre-norm, x += m mixer(norm1(x)); x += m ff(norm2(x)), with one multiplier
m for the whole model and RMS norms taken in groups; its mixer is a talking-heads attention whose
values are its keys ("attention"), an HGRN2 recurrence ("hgrn2"), or attention over a cached
latent with a turned part ("latent_attention"); its feed-forward is a gated MLP or absent.  A run
of consecutive layers may be repeated several times with the same weights (`loop`); ahead of every
pass the stream is remade from itself and the embedding output.  Every size and every constant
that may differ between models comes from the file:

    {"architecture": "Buborax", "vocab": V, "width": E, "residual_mult": m,
     "norm": {"eps": e, "groups": g},
     "loop": {"start": a, "stop": b, "times": n},            (optional)
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "hgrn2", "mixer": {"heads", "dim", "vdim"}, "mlp": null},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask": {"size"},
                           "rot": {"base", "dims"}}, "mlp": {...}}]}

`mask` may be left out: the whole past is then visible.  An optional `max_positions` bounds a
request's length (positions are computed, not looked up).
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, get_float, get_int, get_str

LAYER_TYPES = ("attention", "hgrn2", "latent_attention")
DEFAULT_MAX_POSITIONS = 1 << 16


def _window(m, where):
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object with 'size'")
    return get_int(mask, "size", minimum=1)


def _mask_dict(window):
    return {} if window is None else {"mask": {"size": window}}


@dataclass(frozen=True)
class TalkingMixer:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: Optional[int]

    @classmethod
    def read(cls, m, where):
        heads, kv = get_int(m, "heads", minimum=1), get_int(m, "kv_heads", minimum=1)
        if heads % kv:
            raise ConfigError(f"config.json: key 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
        dim = get_int(m, "dim", minimum=1)
        vdim = get_int(m, "vdim", default=dim, minimum=1)
        if vdim != dim:
            raise ConfigError(f"config.json: key 'vdim' ({vdim}) must equal 'dim' ({dim}): the values are the keys")
        return cls(heads, kv, dim, get_float(m, "scale", positive=True), _window(m, where))

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.dim,
                "scale": self.scale, **_mask_dict(self.window)}


@dataclass(frozen=True)
class RowGatedMixer:
    heads: int
    dim: int
    vdim: int

    @classmethod
    def read(cls, m, where):
        return cls(get_int(m, "heads", minimum=1), get_int(m, "dim", minimum=1), get_int(m, "vdim", minimum=1))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_dims: int
    rot_base: float

    @classmethod
    def read(cls, m, where):
        rot_dim = get_int(m, "rot_dim", default=0, minimum=0)
        dims, base = 0, 10000.0
        if rot_dim:
            rot = m.get("rot")
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
            dims, base = get_int(rot, "dims", default=rot_dim, minimum=0), get_float(rot, "base", positive=True)
            if dims > rot_dim or dims % 2:
                raise ConfigError(f"config.json: key 'dims' ({dims}) must be even and at most 'rot_dim' ({rot_dim})")
        return cls(get_int(m, "heads", minimum=1), get_int(m, "dim", minimum=1), rot_dim, get_int(m, "vdim", minimum=1),
                   get_int(m, "kv_rank", minimum=1), get_float(m, "scale", positive=True), _window(m, where), dims, base)

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale, **_mask_dict(self.window)}
        if self.rot_dim:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


_MIXERS = {"attention": TalkingMixer, "hgrn2": RowGatedMixer, "latent_attention": LatentMixer}


@dataclass(frozen=True)
class BuboraxLayer:
    type: str
    mixer: object                     # TalkingMixer | RowGatedMixer | LatentMixer
    ff: Optional[int]                 # the feed-forward's inner width; None: no feed-forward

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class LayerLoop:
    start: int
    stop: int
    times: int

    def to_dict(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class BuboraxConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    layers: Tuple[BuboraxLayer, ...]
    loop: Optional[LayerLoop] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None
    architecture: str = "Buborax"

    @classmethod
    def from_dict(cls, d):
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: key 'norm' must be an object with 'eps' and 'groups'")
        width = get_int(d, "width", minimum=1)
        groups = get_int(norm, "groups", default=1, minimum=1)
        if width % groups:
            raise ConfigError(f"config.json: key 'width' ({width}) must be a multiple of norm 'groups' ({groups})")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = get_str(entry, "type", choices=set(LAYER_TYPES))
            mlp, ff = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object")
                get_str(mlp, "kind", choices={"dense"})
                ff = get_int(mlp, "ff", minimum=1)
            try:
                mixer = _MIXERS[kind].read(entry["mixer"], where + ".mixer")
            except ConfigError as e:
                raise ConfigError(f"{e} (in {where}.mixer)") from None
            layers.append(BuboraxLayer(kind, mixer, ff))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            if not isinstance(lp, dict):
                raise ConfigError("config.json: key 'loop' must be null or an object with 'start', 'stop', 'times'")
            loop = LayerLoop(get_int(lp, "start", minimum=0), get_int(lp, "stop", minimum=1), get_int(lp, "times", minimum=1))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not lie within the {len(layers)} layers")
        return cls(vocab=get_int(d, "vocab", minimum=1), width=width, norm_eps=get_float(norm, "eps", positive=True),
                   norm_groups=groups, residual_mult=get_float(d, "residual_mult", default=1.0), layers=tuple(layers),
                   loop=loop, max_positions=get_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
                   eos_token_id=get_int(d, "eos_token_id", default=None))

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
