"""Feed-forward parts."""
import torch

from .base import Part
from .linear import Linear, declare_linear
from .plan import WeightDecl
from .registry import register_part


@register_part("feed_forward", "mlp")
class MLP(Part):
    """residual += act(h·W_up + b_up)·W_down + b_down
    (reference src/gpt2.c:283-292; activation src/ops.c:233-241).
    params: size, inner_size, activation ("gelu_tanh" | "gelu_erf" | "xielu" | "relu2", the square of relu), bias,
    weight_layout ("conv1d" = [in,out] in the file, "linear" = [out,in]).
    "xielu" carries two numbers (p, q) of its own in a tensor `act_params`:
    act(z) = softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 otherwise."""

    @classmethod
    def declare_weights(cls, params):
        lay, bias = params.get("weight_layout", "linear"), params.get("bias", True)
        up = declare_linear(params["size"], params["inner_size"], lay, bias)
        down = declare_linear(params["inner_size"], params["size"], lay, bias, init="residual_matrix")
        d = {"up_" + k: v for k, v in up.items()}
        d.update({"down_" + k: v for k, v in down.items()})
        if params["activation"] == "xielu":
            d["act_params"] = WeightDecl((2,), "bias")
        return d

    def load(self, tensors, store):
        lay = self.params.get("weight_layout", "linear")
        self.up = Linear.from_refs(store, tensors["up_weight"], tensors.get("up_bias"), lay)
        self.down = Linear.from_refs(store, tensors["down_weight"], tensors.get("down_bias"), lay)
        self.act_params = self.act_slot = None
        if self.params["activation"] == "xielu":
            from ..csrc import ops
            import math
            p, q = (float(v) for v in tensors["act_params"].tensor.double().tolist())
            softplus = lambda v: max(v, 0.0) + math.log1p(math.exp(-abs(v)))
            self.act_params = (softplus(p), 0.5 + softplus(q))
            if self.rt is not None:
                libs = ["gemm_simt"] + (["gemm_tc", "gemm_few"] if self.rt.dtype == "bfloat16" else [])
                self.act_slot = ops.register_act_params(*self.act_params, libs)

    act_params = act_slot = None

    def workspace_per_token(self):
        act = 4 if self.rt.dtype == "float32" else 2
        return (act + (4 if self.params["activation"] == "xielu" else 0)) * self.params["inner_size"]

    def act_in_own_kernel(self):
        """An activation with numbers of its own is applied in the up-projection's epilogue from a
        slot of the kernel libraries' parameter tables; only a model with more such activations
        than slots sends the product's 32-bit result through a kernel of the activation."""
        return self.params["activation"] == "xielu" and self.act_slot is None

    def forward(self, ctx, h, residual, out=None):
        from ..csrc import ops
        T = h.shape[0]
        u = ctx.alloc((T, self.params["inner_size"]), self.rt.act_dtype)
        if self.act_in_own_kernel():
            z = ctx.alloc((T, self.params["inner_size"]), torch.float32)
            self.up.forward(ctx, h, out=z)
            ops.xielu(z, u, *self.act_params)
        elif self.act_slot is not None:
            self.up.forward(ctx, h, out=u, act=(self.params["activation"], self.act_slot))
        else:
            self.up.forward(ctx, h, out=u, act=self.params["activation"])
        return self.down.forward(ctx, u, out=out, residual=residual)


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """residual += m (act(h Wg^T + bg) * (h Wu^T + bu)) Wd^T + bd.  Gate and up projections are one
    product; the gating runs on its result; the down projection adds into the stream.  The
    multiplier m of the sublayer's result is taken by the gating kernel, in 32-bit, ahead of the
    down projection (which is linear), so a model with m != 1 and a down bias is not served.
    params: size, inner_size, bias, activation ("silu", the default, or "gelu_tanh"), out_mult (m,
    default 1)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        from ..csrc import ops
        if self.params.get("activation", "silu") not in ops.GATE_ACTS:
            raise ValueError(f"gated_mlp: activation {self.params['activation']!r}; known: {sorted(ops.GATE_ACTS)}")
        if float(self.params.get("out_mult", 1.0)) != 1.0 and self.params.get("bias", True):
            raise ValueError("gated_mlp: a result multiplier does not go with a bias on the down projection")

    @classmethod
    def declare_weights(cls, params):
        E, F, bias = params["size"], params["inner_size"], params.get("bias", True)
        d = {"gate_weight": WeightDecl((F, E), "matrix"), "up_weight": WeightDecl((F, E), "matrix"),
             "down_weight": WeightDecl((E, F), "residual_matrix")}
        if bias:
            d.update({"gate_bias": WeightDecl((F,), "bias"), "up_bias": WeightDecl((F,), "bias"),
                      "down_bias": WeightDecl((E,), "bias")})
        return d

    def load(self, tensors, store):
        g, u = tensors["gate_weight"], tensors["up_weight"]
        w = store.computed(g.name + "+" + u.name, lambda: torch.cat([g.tensor.float(), u.tensor.float()], 0))
        b = None
        if "gate_bias" in tensors:
            bg, bu = tensors["gate_bias"], tensors["up_bias"]
            b = store.computed(bg.name + "+" + bu.name, kind="vector",
                               make=lambda: torch.cat([bg.tensor.float(), bu.tensor.float()]))
        self.gate_up = Linear(w, b)
        self.down = Linear(store.matrix(tensors["down_weight"]),
                           store.vector(tensors["down_bias"]) if "down_bias" in tensors else None)

    def workspace_per_token(self):
        return (4 if self.rt.dtype == "float32" else 2) * 3 * self.params["inner_size"] + 512

    def forward(self, ctx, h, residual, out=None):
        from ..csrc import ops
        T, F = h.shape[0], self.params["inner_size"]
        gu = ctx.alloc((T, 2 * F), self.rt.act_dtype)
        self.gate_up.forward(ctx, h, out=gu)
        z = ctx.alloc((T, F), self.rt.act_dtype)
        ops.gated_act(gu, z, act=self.params.get("activation", "silu"), mult=float(self.params.get("out_mult", 1.0)))
        return self.down.forward(ctx, z, out=out, residual=residual)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of `n_experts` small gated feed-forwards without biases, of which a token uses
    `top`: residual += sum over the chosen e of w_e * Wd_e (silu(Wg_e h) * (Wu_e h)).
    Routing: s = sigmoid(h Wr^T) in 32-bit; the choice goes by s + correction, the weights are s
    itself (not renormalised); experts form `n_groups` equal groups of neighbours, a group scores
    the sum of its two largest choice scores, and only experts of the `keep` best groups can be
    chosen (the others count as minus infinity).
    All experts' gate and up matrices are one product over the step's rows; the gating multiplies
    each expert's block of columns by the token's weight for it, which is zero for an expert not
    chosen; the down matrices, side by side, are one product whose contraction is the sum over
    experts.  A step does the same launches whatever the routing says.
    Other routings by parameter: `score` "softmax" (s = softmax over all experts instead of the
    sigmoid), `renorm` (the chosen scores divided by their sum + 1e-20), `weight_scale` (a factor
    of every weight), `correction` false (no such tensor).  `shared_inner_size`: one more expert of
    that inner width (`shared_gate`, `shared_up`, `shared_down`) that every token uses with weight
    1; its matrices lie behind the routed experts' in the same two products.
    params: size, inner_size (an expert's), n_experts, top, n_groups, keep, score, renorm,
    weight_scale, correction, shared_inner_size."""

    @classmethod
    def declare_weights(cls, params):
        E, F, X = params["size"], params["inner_size"], params["n_experts"]
        d = {"router": WeightDecl((X, E), "matrix")}
        if params.get("correction", True):
            d["correction"] = WeightDecl((X,), "bias")
        for e in range(X):
            d.update({f"gate_{e}": WeightDecl((F, E), "matrix"), f"up_{e}": WeightDecl((F, E), "matrix"),
                      f"down_{e}": WeightDecl((E, F), "residual_matrix")})
        Fs = params.get("shared_inner_size")
        if Fs:
            d.update({"shared_gate": WeightDecl((Fs, E), "matrix"), "shared_up": WeightDecl((Fs, E), "matrix"),
                      "shared_down": WeightDecl((E, Fs), "residual_matrix")})
        return d

    def load(self, tensors, store):
        X = self.params["n_experts"]
        gates, ups, downs = ([tensors[f"{k}_{e}"] for e in range(X)] for k in ("gate", "up", "down"))
        if self.params.get("shared_inner_size"):
            gates, ups, downs = gates + [tensors["shared_gate"]], ups + [tensors["shared_up"]], downs + [tensors["shared_down"]]
        self.gate_up = Linear(store.computed("+".join(r.name for r in gates + ups),
                                             lambda: torch.cat([r.tensor.float() for r in gates + ups], 0)), None)
        self.down = Linear(store.computed("|".join(r.name for r in downs),
                                          lambda: torch.cat([r.tensor.float() for r in downs], 1)), None)
        rw = tensors["router"]
        pad = (-X) % 8
        self.router = Linear(store.computed(rw.name + f"+{pad}", lambda: torch.cat(
            [rw.tensor.float(), torch.zeros(pad, rw.tensor.shape[1])], 0)), None)
        self.correction = store.vector(tensors["correction"]) if "correction" in tensors else None

    def workspace_per_token(self):
        p = self.params
        act = 4 if self.rt.dtype == "float32" else 2
        X = p["n_experts"]
        return act * 3 * (X * p["inner_size"] + int(p.get("shared_inner_size") or 0)) + 4 * (2 * X + 8) + 8 * p["top"] + 1024

    def forward(self, ctx, h, residual, out=None):
        from ..csrc import ops
        p = self.params
        T, F, X, top = h.shape[0], p["inner_size"], p["n_experts"], p["top"]
        z = ctx.alloc((T, self.router.out_size), torch.float32)
        self.router.forward(ctx, h, out=z)
        dense = ctx.alloc((T, X), torch.float32)
        ids = ctx.alloc((T, top), torch.int32)
        wts = ctx.alloc((T, top), torch.float32)
        renorm = bool(p.get("renorm", False))
        ops.router(ctx.columns(z, 0, X), self.correction, dense, ids, wts, top, p.get("n_groups", 1), p.get("keep", 1),
                   renorm=renorm, weight_scale=float(p.get("weight_scale", 1.0)), score=p.get("score", "sigmoid"),
                   renorm_eps=1e-20 if renorm else 0.0)
        Fall = X * F + int(p.get("shared_inner_size") or 0)      # the shared expert's columns take weight 1
        gu = ctx.alloc((T, 2 * Fall), self.rt.act_dtype)
        self.gate_up.forward(ctx, h, out=gu)
        a = ctx.alloc((T, Fall), self.rt.act_dtype)
        ops.gated_act(gu, a, weights=dense, per=F, n_weighted=X * F)
        return self.down.forward(ctx, a, out=out, residual=residual)
