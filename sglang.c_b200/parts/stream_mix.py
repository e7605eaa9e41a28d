"""Parts that mix the residual streams of several depths."""
import torch

from ..csrc import ops
from .base import Part
from .plan import WeightDecl
from .registry import register_part


@register_part("stream_mix", "depth_weighted_average")
class DepthWeightedAverage(Part):
    """With X_0 the embedding output and X_(i+1) the result of layer i, what leaves layer i is
    sum_{j=0..i+1} w[j] * X_j, w being this layer's own i+2 weights.  The X_j of the step's
    tokens are kept, 32-bit, in one buffer of the step workspace that the first layer takes
    (`begin`, ahead of the block's own buffers) and every layer adds to (`finish`).
    params: index (i), n_layers, size."""

    @classmethod
    def declare_weights(cls, params):
        return {"weights": WeightDecl((params["index"] + 2,), "norm_gain")}

    def load(self, tensors, store):
        self.weights = store.vector(tensors["weights"])

    def workspace_per_token(self):
        return 4 * self.params["size"] * (self.params["n_layers"] + 1)

    def begin(self, ctx, x):
        if self.params["index"] == 0:
            hist = ctx.alloc((self.params["n_layers"] + 1,) + tuple(x.shape), torch.float32)
            ctx.shared["depth_streams"] = hist
            ops.depth_mix(x, hist, 1, None)

    def terms(self, ctx):
        """(streams kept so far, terms of this layer's sum, its weights): for a kernel that does
        the mix itself, in place of finish()."""
        return ctx.shared["depth_streams"], self.params["index"] + 2, self.weights

    def finish(self, ctx, x):
        ops.depth_mix(x, ctx.shared["depth_streams"], self.params["index"] + 2, self.weights)
        return x


@register_part("stream_mix", "input_reentry")
class InputReentry(Part):
    """Ahead of pass t of a group of layers that runs several times over with the same weights, the
    stream is remade from itself and the embedding output X_0 of the same tokens:
        x <- W [x ; X_0] + step[t]        (W [size, 2 size], x's columns first; step [times, size]).
    `start` (after the embedding) takes a buffer of 2 size columns in the activation precision
    from the step workspace, below the layers' buffers, and puts X_0 into its right half once;
    `enter` puts x into the left half and runs the product, whose 32-bit result replaces x, with
    step[t] as its bias.  params: size, times."""

    @classmethod
    def declare_weights(cls, params):
        E = params["size"]
        return {"in_weight": WeightDecl((E, 2 * E), "carry"), "steps": WeightDecl((params["times"], E), "bias")}

    def load(self, tensors, store):
        from .linear import Linear
        self.inp = Linear(store.matrix(tensors["in_weight"]), None)
        steps = store.vector(tensors["steps"])
        self.steps = [steps[t] for t in range(self.params["times"])]

    def workspace_per_token(self):
        return (4 if self.rt.dtype == "float32" else 2) * 2 * self.params["size"] + 256

    def start(self, ctx, x):
        E = self.params["size"]
        rows = ctx.alloc((x.shape[0], 2 * E), self.rt.act_dtype)
        ctx.shared[("input_reentry", id(self))] = rows
        ops.cast_rows(x, ctx.columns(rows, E, 2 * E))

    def enter(self, ctx, x, t):
        rows = ctx.shared[("input_reentry", id(self))]
        ops.cast_rows(x, ctx.columns(rows, 0, self.params["size"]))
        ctx.rt.gemm(rows, self.inp.weight, self.steps[t], out=x, few_ok=ctx.few_token_ok)
        return x


@register_part("stream_mix", "token_gated_input")
class TokenGatedInput(Part):
    """An input from a second token table, gated by the stream and added to it behind a norm:
        e = table[token][index * dim : (index + 1) * dim]      (the table holds every layer's part)
        g = gelu_tanh(Wg x) * e;   y = Wp g;   x += y / sqrt(mean(y^2) + eps) * gain
    Two small products with 32-bit results, the gate and gather between them, and the norm that
    sums into the 32-bit stream.  params: size, dim, index, n_layers, vocab_size, eps."""

    @classmethod
    def declare_weights(cls, params):
        E, d = params["size"], params["dim"]
        return {"table": WeightDecl((params["vocab_size"], params["n_layers"] * d), "embedding"),
                "gate_weight": WeightDecl((d, E), "matrix"), "proj_weight": WeightDecl((E, d), "residual_matrix"),
                "norm": WeightDecl((E,), "norm_gain")}

    def load(self, tensors, store):
        from .linear import Linear
        self.table = store.matrix(tensors["table"])
        self.gate = Linear(store.matrix(tensors["gate_weight"]), None)
        self.proj = Linear(store.matrix(tensors["proj_weight"]), None)
        self.gain = store.vector(tensors["norm"])

    def workspace_per_token(self):
        act = 4 if self.rt.dtype == "float32" else 2
        return (4 + act) * self.params["dim"] + 512

    def finish(self, ctx, x, h=None, y=None, cast_out=None):
        """x += the gated input.  h: the stream's rows in the products' precision, if the caller has
        them; y: a 32-bit buffer [T, size] to use; cast_out: a buffer that takes the new rows in its
        own precision (same launch as the sum)."""
        p = self.params
        T, d = x.shape[0], p["dim"]
        if h is None:
            if self.rt.act_dtype == torch.float32:
                h = x
            else:
                h = ctx.alloc((T, p["size"]), self.rt.act_dtype)
                ops.cast_rows(x, h)
        if y is None:
            y = ctx.alloc((T, p["size"]), torch.float32)
        z = ctx.alloc((T, d), torch.float32)
        self.gate.forward(ctx, h, out=z)
        g = ctx.alloc((T, d), self.rt.act_dtype)
        ops.gated_gather(z, ctx.tokens, self.table, p["index"] * d, g, err_flag=ctx.err_flag)
        self.proj.forward(ctx, g, out=y)
        if cast_out is not None and x.is_contiguous():
            ops.norm_add_tail(y, self.gain, float(p["eps"]), x, form="rms", then=(None, 0.0, "copy", cast_out))
        else:
            ops.norm_rows(y, self.gain, None, float(p["eps"]), x[:T], form="rms", add=True)
            if cast_out is not None:
                ops.cast_rows(x[:T], cast_out)
        return x
