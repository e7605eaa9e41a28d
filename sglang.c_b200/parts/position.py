"""Position encodings.  A position part can act at the embedding (a table added
to the token rows), inside a mixer (a change of queries and keys), or both."""
from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


class PositionEncoding(Part):
    def additive_table(self):
        return None

    def apply_embedding(self, ctx, x):
        pass

    def rotate(self, ctx, q, k):
        pass


@register_part("position", "none")
class NoPositions(PositionEncoding):
    pass


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    """x[t,:] += table[pos[t],:]  (reference src/gpt2.c:212-216).
    params: max_positions, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"table": WeightDecl((params["max_positions"], params["size"]), "embedding")}

    def load(self, tensors, store):
        self.table = store.matrix(tensors["table"])

    def additive_table(self):
        return self.table

    def apply_embedding(self, ctx, x):
        ops.add_rows(x, ctx.positions, self.table)


@register_part("position", "sinusoidal")
class SinusoidalPositions(PositionEncoding):
    """A fixed vector added at the embedding, computed from the position, no table and no
    bound: entry 2i is sin(p * base^(-2i/size)), entry 2i+1 the cosine of the same angle.
    The inverse wavelengths are made once, in 64-bit; the embedding kernel forms the angle.
    params: size, base."""

    def load(self, tensors, store):
        import torch
        size, base = int(self.params["size"]), float(self.params["base"])
        i = torch.arange((size + 1) // 2, dtype=torch.float64)
        self.inv_freq = (base ** (-2.0 * i / size)).contiguous().to(self.rt.device)

    def inverse_wavelengths(self):
        return self.inv_freq


@register_part("position", "rotary")
class RotaryPositions(PositionEncoding):
    """Rotary positions inside a mixer: the first `dims` entries of every query and key head are
    turned in pairs (i, i + dims/2) by the angle position * f_i, f_i = base^(-2i/dims).
    With `scaling` = {factor, original, fast, slow} (YaRN) a pair's frequency is blended between
    f_i and f_i / factor: with pair(t) = dims ln(original / (2 pi t)) / (2 ln base) the pair index at
    which `original` positions make t turns, lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are both multiplied by
    0.1 ln(factor) + 1.  The table is made once, in 64-bit; the mixer's kernel forms the angles.
    A mixer builds this part from its own params (a model may turn each layer differently).
    `pairing` "neighbours" pairs entry 2i with 2i+1 instead (for the kernels that take the choice).
    params: dims, base, scaling (None or the four numbers), pairing ("halves", the default, or
    "neighbours")."""

    def load(self, tensors, store):
        import math

        import torch
        dims, base, sc = int(self.params["dims"]), float(self.params["base"]), self.params.get("scaling")
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = base ** (-2.0 * i / dims) if dims else i
        self.multiplier = 1.0
        if sc and dims:
            factor, orig = float(sc["factor"]), float(sc["original"])
            pair = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            lo = max(math.floor(pair(float(sc["fast"]))), 0)
            hi = min(math.ceil(pair(float(sc["slow"]))), dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.multiplier = 0.1 * math.log(factor) + 1.0
        self.frequencies = f.contiguous().to(self.rt.device) if self.rt is not None else f
        self.dims = dims
        self.pairing = self.params.get("pairing", "halves")
        if self.pairing not in ("halves", "neighbours"):
            raise ValueError(f"rotary: pairing {self.pairing!r}; known: halves, neighbours")
