"""Arrangements of norm, mixer and feed-forward around the residual stream."""
import torch

from .base import Part
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (reference src/gpt2.c:219-293).
    The residual stream x stays 32-bit; the normalised rows are in the
    runtime's activation precision.  The second sublayer is there only if the layer has an
    `ffn`.  (A model that multiplies every sublayer's result by a constant gives that constant
    to the sublayers' parts, which take it ahead of their last product.)"""

    def workspace_per_token(self, layer):
        act = 4 if self.rt.dtype == "float32" else 2
        inner = layer.mixer.workspace_per_token()
        if "ffn" in layer.parts:
            inner = max(inner, layer.ffn.workspace_per_token())
        return act * layer.norm1.params["size"] + inner

    def forward(self, ctx, x, layer, cache, position=None):
        T = x.shape[0]
        mark = ctx.mark()
        h = ctx.alloc((T, x.shape[1]), self.rt.act_dtype)
        layer.norm1.forward(ctx, x, h)
        inner = ctx.mark()
        layer.mixer.forward(ctx, h, residual=x, cache=cache, position=position)
        ctx.release(inner)               # the mixer's buffers make room for the feed-forward's
        if "ffn" in layer.parts:
            layer.norm2.forward(ctx, x, h)
            layer.ffn.forward(ctx, h, residual=x)
        ctx.release(mark)
        return x


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Part):
    """A norm ahead of and a norm behind each sublayer:
    x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))).  The second sublayer is there
    only if the layer has an `ffn`.  A sublayer's result is a 32-bit buffer; the norm behind it
    sums it into the 32-bit stream in the same kernel.  A layer with a `depth_mix` sub-part
    (category stream_mix) hands x to it before and after."""

    MIX_IN_TAIL_MAX_ROWS = 256

    def workspace_per_token(self, layer):
        act = 4 if self.rt.dtype == "float32" else 2
        E = layer.norm1.params["size"]
        inner = layer.mixer.workspace_per_token()
        if "ffn" in layer.parts:
            inner = max(inner, layer.ffn.workspace_per_token())
        extra = layer.depth_mix.workspace_per_token() if "depth_mix" in layer.parts else 0
        return (act + 4) * E + inner + extra

    def forward(self, ctx, x, layer, cache, position=None):
        T, E = x.shape
        mix = layer.parts.get("depth_mix")
        if mix is not None:
            mix.begin(ctx, x)                # what it keeps for the step lies below the layers' buffers
        mark = ctx.mark()
        h = ctx.alloc((T, E), self.rt.act_dtype)
        y = ctx.alloc((T, E), torch.float32)
        layer.norm1.forward(ctx, x, h)
        inner = ctx.mark()
        layer.mixer.forward(ctx, h, residual=None, cache=cache, position=position, out=y)
        ctx.release(inner)
        # the norm behind a sublayer takes the next step along in its launch: the norm ahead of the
        # feed-forward, or (behind the layer's last sublayer) the depth mix
        # (the mix joins that launch in steps of few rows, where a launch costs more than its bytes;
        # over many rows the mix's own kernel streams the kept results several times faster)
        has_ffn = "ffn" in layer.parts
        terms = mix.terms(ctx) if mix is not None and T <= self.MIX_IN_TAIL_MAX_ROWS else None
        done = layer.norm1b.add_into(ctx, y, x, then=(layer.norm2, h) if has_ffn else None,
                                     mix=None if has_ffn else terms)
        if has_ffn:
            if not done:
                layer.norm2.forward(ctx, x, h)
            layer.ffn.forward(ctx, h, residual=None, out=y)
            ctx.release(inner)
            done = layer.norm2b.add_into(ctx, y, x, mix=terms)
        ctx.release(mark)
        if mix is not None and not done:
            mix.finish(ctx, x)
        return x


@register_part("block", "parallel_sublayers")
class ParallelSublayersBlock(Part):
    """One norm, both sublayers read it: h = norm1(x); x += mixer(h) + ffn(h).  The feed-forward
    is there only if the layer has an `ffn`.  Each sublayer's last product adds into the 32-bit
    stream from its epilogue (or, for a mixer that normalises its result, from that norm)."""

    def workspace_per_token(self, layer):
        act = 4 if self.rt.dtype == "float32" else 2
        inner = layer.mixer.workspace_per_token()
        if "ffn" in layer.parts:
            inner = max(inner, layer.ffn.workspace_per_token())
        return act * layer.norm1.params["size"] + inner

    def forward(self, ctx, x, layer, cache, position=None):
        T = x.shape[0]
        mark = ctx.mark()
        h = ctx.alloc((T, x.shape[1]), self.rt.act_dtype)
        layer.norm1.forward(ctx, x, h)
        inner = ctx.mark()
        layer.mixer.forward(ctx, h, residual=x, cache=cache, position=position)
        ctx.release(inner)
        if "ffn" in layer.parts:
            layer.ffn.forward(ctx, h, residual=x)
        ctx.release(mark)
        return x


@register_part("block", "post_norm")
class PostNormBlock(Part):
    """A norm on each sublayer's result only; the sublayers read the stream itself:
    x += norm1(mixer(x)); x += norm2(ffn(x)) (the second only if the layer has an `ffn`); then, if
    the layer has a `side` sub-part (category stream_mix), x = side.finish(x) (an input that is made
    from the stream and the step's tokens and added to it).  A sublayer's result is a 32-bit buffer;
    the norm behind it sums it into the 32-bit stream.  In a runtime whose products take another
    precision than the stream's, the stream's rows in that precision are written by the same launch
    that last changed them (and kept in ctx.shared for the next layer of this kind), so that every
    product reads rows that are up to date without a launch of its own.
    params: last (the model's last layer: nobody reads the stream's rows in the products'
    precision after it)."""

    KEY = "post_norm_rows"

    def workspace_per_token(self, layer):
        act = 4 if self.rt.dtype == "float32" else 2
        E = layer.norm1.params["size"]
        inner = layer.mixer.workspace_per_token()
        if "ffn" in layer.parts:
            inner = max(inner, layer.ffn.workspace_per_token())
        if "side" in layer.parts:
            inner = max(inner, layer.side.workspace_per_token())
        return (act + 4) * E + 256 + inner

    def forward(self, ctx, x, layer, cache, position=None):
        from ..csrc import ops
        T, E = x.shape
        mark = ctx.mark()
        same = self.rt.act_dtype == torch.float32
        if same:
            h = x                              # the products read the stream as it is
        else:
            h = ctx.alloc((T, E), self.rt.act_dtype)
            if ctx.shared.get(self.KEY) is not h:      # (the layer before did not leave them)
                ops.cast_rows(x, h)
        y = ctx.alloc((T, E), torch.float32)
        inner = ctx.mark()
        has_ffn, has_side = "ffn" in layer.parts, "side" in layer.parts
        read_again = lambda more: None if same or not more else h
        layer.mixer.forward(ctx, h, residual=None, cache=cache, position=position, out=y)
        ctx.release(inner)
        keep = has_ffn or has_side or not self.params.get("last")
        self._add(ctx, layer.norm1, y, x, read_again(keep))
        if has_ffn:
            layer.ffn.forward(ctx, h, residual=None, out=y)
            ctx.release(inner)
            keep = has_side or not self.params.get("last")
            self._add(ctx, layer.norm2, y, x, read_again(keep))
        if has_side:
            layer.side.finish(ctx, x, h=h, y=y, cast_out=read_again(not self.params.get("last")))
            ctx.release(inner)
        ctx.shared[self.KEY] = None if same or self.params.get("last") else h
        ctx.release(mark)
        return x

    @staticmethod
    def _add(ctx, norm, y, x, cast_out):
        if cast_out is None:
            norm.add_into(ctx, y, x)
        else:
            norm.add_into(ctx, y, x, then_cast=cast_out)
