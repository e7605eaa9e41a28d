"""Recurrent mixers: a state of fixed size per request, in a slot of the cache manager."""
import torch

from ..cache.needs import CacheNeed
from ..csrc import ops
from .base import Part
from .linear import Linear
from .plan import WeightDecl
from .registry import register_part


@register_part("mixer", "min_gru")
class MinGRU(Part):
    """A gated recurrence whose gates read the current token only:
    z = sigmoid(h·Wzᵀ + bz), u = h·Wxᵀ + bx, candidate c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z) S_(t-1) + z c, element by element; out = (S_t * silu(h·Wgᵀ))·Woᵀ.
    The three input projections are one product whose 32-bit result the scan kernel reads;
    gates, candidate and state are 32-bit; the state (`width` floats) starts at zero and is
    carried per request.  params: size, width."""

    @classmethod
    def declare_weights(cls, params):
        E, W = params["size"], params["width"]
        return {"gate_weight": WeightDecl((W, E), "matrix"), "gate_bias": WeightDecl((W,), "bias"),
                "cand_weight": WeightDecl((W, E), "matrix"), "cand_bias": WeightDecl((W,), "bias"),
                "out_gate_weight": WeightDecl((W, E), "matrix"),
                "out_weight": WeightDecl((E, W), "residual_matrix")}

    def load(self, tensors, store):
        W = self.params["width"]
        names = [tensors[k] for k in ("gate_weight", "cand_weight", "out_gate_weight")]
        w = store.computed("+".join(r.name for r in names), lambda: torch.cat([r.tensor.float() for r in names], 0))
        bz, bx = tensors["gate_bias"], tensors["cand_bias"]
        b = store.computed(bz.name + "+" + bx.name + "+0", kind="vector",
                           make=lambda: torch.cat([bz.tensor.float(), bx.tensor.float(), torch.zeros(W)]))
        self.inp = Linear(w, b)
        self.out = Linear(store.matrix(tensors["out_weight"]), None)

    def cache_need(self):
        return CacheNeed.state((self.params["width"],), "float32")

    def workspace_per_token(self):
        act = 4 if self.rt.dtype == "float32" else 2
        # the projections, the gated state, and (steps with long portions) the chunk sums: two
        # floats a channel for every chunk's worth of tokens and three for every request, of
        # which a step has no more than tokens
        W = self.params["width"]
        return W * (12 + act) + 12 * W + 8 * W // ops.GATED_SCAN_PIECE + 8

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        T, W = h.shape[0], self.params["width"]
        pre = ctx.alloc((T, 3 * W), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        y = ctx.alloc((T, W), self.rt.act_dtype)
        need = ops.mingru_scan_workspace(ctx.R, W, T, ctx.max_q_len)
        ws = ctx.alloc((need,), torch.float32) if need else None
        ops.mingru_scan(ctx.columns(pre, 0, W), ctx.columns(pre, W, 2 * W), ctx.columns(pre, 2 * W, 3 * W), y,
                        cache.tensor, ctx.q_start, ctx.state_slots, ctx.R, ctx.max_q_len, workspace=ws)
        return self.out.forward(ctx, y, out=out, residual=residual)


def _stacked(store, refs):
    """Projections that read the same rows, laid one under the other: one product."""
    return store.computed("+".join(r.name for r in refs), lambda: torch.cat([r.tensor.float() for r in refs], 0))


@register_part("mixer", "gated_delta")
class GatedDeltaRule(Part):
    """The gated delta rule: per head a matrix state S [dim x v_dim] that decays, is corrected
    towards the current value along the current key, and is read with the query:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    q, k (n_qk_heads x dim) and v (n_heads x v_dim) are projections of h that pass a causal
    convolution of `conv` taps over time per channel and silu; q and k are then unit vectors per
    head (eps 1e-6 inside the root), q times dim^(-1/2); head i reads q/k head i / (n_heads /
    n_qk_heads).  beta = sigmoid(h Wb^T); g = exp(-exp(A_log) softplus(h Wa^T + dt_bias)).
    Each head's o is divided by its root mean square (eps), times a gain of v_dim entries shared by
    the heads, times silu(h Wg^T); then the output projection.  All projections are one product
    with a 32-bit result; convolution, gates, state and output stage are 32-bit.  Kept per request:
    S, and the last conv - 1 inputs of the convolution.
    params: size, n_heads, n_qk_heads, dim, v_dim, conv, eps."""

    UNIT_EPS = 1e-6

    @classmethod
    def declare_weights(cls, params):
        E, H, G, D, V, K = (params[k] for k in ("size", "n_heads", "n_qk_heads", "dim", "v_dim", "conv"))
        return {"q_weight": WeightDecl((G * D, E), "matrix"), "q_conv": WeightDecl((G * D, K), "conv_taps"),
                "k_weight": WeightDecl((G * D, E), "matrix"), "k_conv": WeightDecl((G * D, K), "conv_taps"),
                "v_weight": WeightDecl((H * V, E), "matrix"), "v_conv": WeightDecl((H * V, K), "conv_taps"),
                "beta_weight": WeightDecl((H, E), "matrix"), "a_weight": WeightDecl((H, E), "matrix"),
                "A_log": WeightDecl((H,), "bias"), "dt_bias": WeightDecl((H,), "bias"),
                "gate_weight": WeightDecl((H * V, E), "matrix"), "norm": WeightDecl((V,), "norm_gain"),
                "out_weight": WeightDecl((E, H * V), "residual_matrix")}

    def load(self, tensors, store):
        p = self.params
        H, G, D, V = p["n_heads"], p["n_qk_heads"], p["dim"], p["v_dim"]
        refs = [tensors[k] for k in ("q_weight", "k_weight", "v_weight", "gate_weight", "beta_weight", "a_weight")]
        n = 2 * G * D + 2 * H * V + 2 * H
        pad = (-n) % 8                     # whole 32-byte pieces of 32-bit results a row
        self.inp = Linear(store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0)), None)
        conv = [tensors[k] for k in ("q_conv", "k_conv", "v_conv")]
        self.taps = store.computed("+".join(r.name for r in conv), kind="vector",
                                   make=lambda: torch.cat([r.tensor.float() for r in conv], 0))
        self.A_log, self.dt_bias = store.vector(tensors["A_log"]), store.vector(tensors["dt_bias"])
        self.norm = store.vector(tensors["norm"])
        self.out = Linear(store.matrix(tensors["out_weight"]), None)
        self.channels = 2 * G * D + H * V
        self.segments = [(0, G, D, 1, D ** -0.5), (G * D, G, D, 1, 1.0), (2 * G * D, H, V, 0, 1.0)]

    def cache_need(self):
        p = self.params
        C = 2 * p["n_qk_heads"] * p["dim"] + p["n_heads"] * p["v_dim"]
        return (CacheNeed.state((p["n_heads"], p["dim"], p["v_dim"]), "float32"),
                CacheNeed.state((max(p["conv"] - 1, 0), C), "float32"))

    def workspace_per_token(self):
        p = self.params
        H, G, D, V = p["n_heads"], p["n_qk_heads"], p["dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        return 4 * (2 * G * D + 2 * H * V + 2 * H + 8) + 4 * (2 * G * D + H * V) + 8 * H + 4 * H * V + act * H * V + 2048

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, G, D, V = p["n_heads"], p["n_qk_heads"], p["dim"], p["v_dim"]
        T, C = h.shape[0], self.channels
        state, tail = cache
        pre = ctx.alloc((T, self.inp.out_size), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        y = ctx.alloc((T, C), torch.float32)
        gates = ctx.alloc((T, 2 * H), torch.float32)
        gate_col = C + H * V
        ops.short_conv(pre, self.taps, tail.tensor, y, ctx.token_req, ctx.q_start, ctx.state_slots, ctx.R,
                       self.segments, unit_eps=self.UNIT_EPS,
                       gates=(H, gate_col, gate_col + H, self.A_log, self.dt_bias, gates))
        o = ctx.alloc((T, H * V), torch.float32)
        ops.matrix_state("delta", ctx.columns(y, 0, G * D), ctx.columns(y, G * D, 2 * G * D), ctx.columns(y, 2 * G * D, C),
                         o, state.tensor, ctx.q_start, ctx.state_slots, ctx.R, H, G, D, V, gates=gates)
        z = ctx.alloc((T, H * V), self.rt.act_dtype)
        ops.gated_norm(o, ctx.columns(pre, C, C + H * V), self.norm, z, H, V, float(p["eps"]), "silu")
        return self.out.forward(ctx, z, out=out, residual=residual)


@register_part("mixer", "linear_decay_attention")
class LinearDecayAttention(Part):
    """Linear attention with a fixed decay per head (lightning attention): q = silu(h Wq^T),
    k = silu(h Wk^T) (n_heads x dim), v = silu(h Wv^T) (n_heads x v_dim); per head
    S <- decay_h S + k v^T, o = S^T q, no other scale.  The heads' results side by side are
    RMS-normed together with a gain, multiplied by sigmoid(h Wg^T) and projected.  The state is
    32-bit, starts at zero and is carried per request.
    params: size, n_heads, dim, v_dim, decay (one number per head), eps."""

    @classmethod
    def declare_weights(cls, params):
        E, H, D, V = (params[k] for k in ("size", "n_heads", "dim", "v_dim"))
        return {"q_weight": WeightDecl((H * D, E), "matrix"), "k_weight": WeightDecl((H * D, E), "matrix"),
                "v_weight": WeightDecl((H * V, E), "matrix"), "gate_weight": WeightDecl((H * V, E), "matrix"),
                "norm": WeightDecl((H * V,), "norm_gain"), "out_weight": WeightDecl((E, H * V), "residual_matrix")}

    def load(self, tensors, store):
        refs = [tensors[k] for k in ("q_weight", "k_weight", "v_weight", "gate_weight")]
        self.inp = Linear(_stacked(store, refs), None)
        self.norm = store.vector(tensors["norm"])
        self.out = Linear(store.matrix(tensors["out_weight"]), None)
        decay = [float(v) for v in self.params["decay"]]
        if len(decay) != self.params["n_heads"]:
            raise ValueError("linear_decay_attention: one decay per head")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(self.rt.device)

    def cache_need(self):
        p = self.params
        return CacheNeed.state((p["n_heads"], p["dim"], p["v_dim"]), "float32")

    def workspace_per_token(self):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        return 4 * (2 * H * D + 2 * H * V) + 4 * H * V + act * H * V + 1024

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        T = h.shape[0]
        pre = ctx.alloc((T, 2 * H * D + 2 * H * V), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        o = ctx.alloc((T, H * V), torch.float32)
        ops.matrix_state("decay", ctx.columns(pre, 0, H * D), ctx.columns(pre, H * D, 2 * H * D),
                         ctx.columns(pre, 2 * H * D, 2 * H * D + H * V), o, cache.tensor, ctx.q_start, ctx.state_slots,
                         ctx.R, H, H, D, V, head_decay=self.decay, silu_in=True)
        z = ctx.alloc((T, H * V), self.rt.act_dtype)
        ops.gated_norm(o, ctx.columns(pre, 2 * H * D + H * V, 2 * H * D + 2 * H * V), self.norm, z, 1, H * V,
                       float(p["eps"]), "sigmoid")
        return self.out.forward(ctx, z, out=out, residual=residual)


@register_part("mixer", "hgrn2")
class RowGatedState(Part):
    """HGRN2: linear attention whose forget gate also says how much is written.  Per head a matrix
    state S [dim x v_dim]; with q = silu(h Wq^T), v = h Wv^T and, per head and row, the gate
    f = l + (1 - l) sigmoid(h Wf^T + bf), l a learned lower bound,
        S <- diag(f) S + (1 - f) v^T;   o = S^T q
    (no key and no other scale).  Each head's o is divided by its root mean square (eps) and
    multiplied by a gain of v_dim entries that the heads share; the heads side by side go through
    the output projection.  The three input projections are one product with a 32-bit result;
    gates, state and the norm are 32-bit.  S starts at zero and is carried per request.
    params: size, n_heads, dim, v_dim, eps, out_mult (a multiplier of the mixer's result, default
    1, folded into the norm's gain)."""

    @classmethod
    def declare_weights(cls, params):
        E, H, D, V = (params[k] for k in ("size", "n_heads", "dim", "v_dim"))
        return {"q_weight": WeightDecl((H * D, E), "matrix"), "gate_weight": WeightDecl((H * D, E), "matrix"),
                "gate_bias": WeightDecl((H * D,), "bias"), "lower": WeightDecl((H * D,), "fraction"),
                "v_weight": WeightDecl((H * V, E), "matrix"), "norm": WeightDecl((V,), "norm_gain"),
                "out_weight": WeightDecl((E, H * V), "residual_matrix")}

    def load(self, tensors, store):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        refs = [tensors[k] for k in ("q_weight", "gate_weight", "v_weight")]
        pad = (-(2 * H * D + H * V)) % 8
        self.inp_w = store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0))
        fb = tensors["gate_bias"]
        bias = store.computed(f"0+{fb.name}+0+{pad}", kind="vector", make=lambda: torch.cat(
            [torch.zeros(H * D), fb.tensor.float(), torch.zeros(H * V + pad)]))
        self.inp = Linear(self.inp_w, bias)
        self.lower = store.vector(tensors["lower"])
        m = float(p.get("out_mult", 1.0))
        g = tensors["norm"]
        self.norm = store.vector(g) if m == 1.0 else store.computed(
            f"{g.name}*{m!r}", kind="vector", make=lambda: (g.tensor.double() * m).float())
        self.out = Linear(store.matrix(tensors["out_weight"]), None)

    def cache_need(self):
        p = self.params
        return CacheNeed.state((p["n_heads"], p["dim"], p["v_dim"]), "float32")

    def workspace_per_token(self):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        return 4 * (2 * H * D + H * V + 8) + 4 * H * V + act * H * V + 1024

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        T = h.shape[0]
        pre = ctx.alloc((T, self.inp.out_size), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        o = ctx.alloc((T, H * V), torch.float32)
        ops.matrix_state("row_gate", ctx.columns(pre, 0, H * D), ctx.columns(pre, H * D, 2 * H * D),
                         ctx.columns(pre, 2 * H * D, 2 * H * D + H * V), o, cache.tensor, ctx.q_start,
                         ctx.state_slots, ctx.R, H, H, D, V, silu_in=True, lower=self.lower)
        z = ctx.alloc((T, H * V), self.rt.act_dtype)
        ops.gated_norm(o, None, self.norm, z, H, V, float(p["eps"]), "none")
        return self.out.forward(ctx, z, out=out, residual=residual)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """Linear attention with a learned decay per key channel and token:
        q = h Wq^T * dim^(-1/2), k = h Wk^T (n_heads x dim), v = h Wv^T (n_heads x v_dim);
        a = sigmoid(z)^(1/tau), z = (h Wa1^T) Wa2^T + ba, laid out n_heads x dim (a low-rank product);
        per head S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t.
    Each head's o is divided by its root mean square (eps) times a gain of v_dim entries that the heads
    share; the heads side by side are multiplied by silu(h Wg^T) and projected.  q, k, v, the gate and
    the decay's first factor are one product with a 32-bit result; the decay's second factor is a
    small product of its own (its input in the activation precision, its bias in the epilogue, a
    32-bit result); decays, state and norm are 32-bit.  S starts at zero and is carried per request.
    params: size, n_heads, dim, v_dim, tau, eps, out_mult (a multiplier of the mixer's result, default
    1, folded into the norm's gain), decay_rank (only for weights made at random: the rank of the
    decay's two factors is what the file's tensors have)."""

    @classmethod
    def declare_weights(cls, params):
        E, H, D, V = (params[k] for k in ("size", "n_heads", "dim", "v_dim"))
        r = -int(params.get("decay_rank", 16))      # free: the file's tensors decide the rank
        return {"q_weight": WeightDecl((H * D, E), "matrix"), "k_weight": WeightDecl((H * D, E), "matrix"),
                "v_weight": WeightDecl((H * V, E), "matrix"), "gate_weight": WeightDecl((H * V, E), "matrix"),
                "decay_down": WeightDecl((r, E), "matrix"), "decay_up": WeightDecl((H * D, r), "matrix"),
                "decay_bias": WeightDecl((H * D,), "bias"), "norm": WeightDecl((V,), "norm_gain"),
                "out_weight": WeightDecl((E, H * V), "residual_matrix")}

    def load(self, tensors, store):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        refs = [tensors[k] for k in ("q_weight", "k_weight", "v_weight", "gate_weight", "decay_down")]
        self.rank = refs[-1].tensor.shape[0]
        if tuple(tensors["decay_up"].tensor.shape) != (H * D, self.rank):
            raise ValueError(f"gated_linear_attention: the decays' factors are [{self.rank}, size] and "
                             f"{list(tensors['decay_up'].tensor.shape)}: their ranks differ")
        n = 2 * H * D + 2 * H * V + self.rank
        pad = (-n) % 8
        self.inp = Linear(store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0)), None)
        self.up = Linear(store.matrix(tensors["decay_up"]), store.vector(tensors["decay_bias"]))
        m = float(p.get("out_mult", 1.0))
        g = tensors["norm"]
        self.norm = store.vector(g) if m == 1.0 else store.computed(
            f"{g.name}*{m!r}", kind="vector", make=lambda: (g.tensor.double() * m).float())
        self.out = Linear(store.matrix(tensors["out_weight"]), None)

    def cache_need(self):
        p = self.params
        return CacheNeed.state((p["n_heads"], p["dim"], p["v_dim"]), "float32")

    def workspace_per_token(self):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        r = getattr(self, "rank", 64)
        return 4 * (2 * H * D + 2 * H * V + r + 8) + act * r + 4 * H * D + 4 * H * V + act * H * V + 2048

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, D, V, r = p["n_heads"], p["dim"], p["v_dim"], self.rank
        T = h.shape[0]
        pre = ctx.alloc((T, self.inp.out_size), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        c_v, c_g, c_a = 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V
        low = ctx.columns(pre, c_a, c_a + r)
        if self.rt.act_dtype != torch.float32:
            low_a = ctx.alloc((T, r), self.rt.act_dtype)
            ops.cast_rows(low, low_a)
            low = low_a
        z = ctx.alloc((T, H * D), torch.float32)
        self.up.forward(ctx, low, out=z)
        o = ctx.alloc((T, H * V), torch.float32)
        ops.matrix_state("row_decay", ctx.columns(pre, 0, H * D), ctx.columns(pre, H * D, 2 * H * D),
                         ctx.columns(pre, c_v, c_g), o, cache.tensor, ctx.q_start, ctx.state_slots, ctx.R, H, H, D, V,
                         row_z=z, tau=float(p["tau"]), q_scale=float(D) ** -0.5)
        y = ctx.alloc((T, H * V), self.rt.act_dtype)
        ops.gated_norm(o, ctx.columns(pre, c_g, c_a), self.norm, y, H, V, float(p["eps"]), "silu")
        return self.out.forward(ctx, y, out=out, residual=residual)


@register_part("mixer", "mlstm")
class MatrixMemory(Part):
    """The matrix memory of xLSTM (mLSTM) with exponential gates and a running maximum:
        q = h Wq^T * dim^(-1/2), k = h Wk^T (n_heads x dim), v = h Wv^T (n_heads x v_dim);
        per head the log gates i = cap tanh((h wi + bi) / cap), f = log sigmoid(cap tanh((h wf + bf) / cap));
        m_t = max(f + m_(t-1), i)                                   (m starts at 0)
        S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,   n_t likewise with k alone;
        o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6).
    Each head's o is divided by its root mean square (eps); the heads side by side are multiplied by a
    gain of n_heads x v_dim entries and by sigmoid(h Wg^T), then projected.  All projections are one
    product with a 32-bit result (the gates' biases in its epilogue); gates, maxima, state and norm
    are 32-bit.  Kept per request: S with n as one more column behind it ([n_heads, dim, v_dim + 1]),
    and m ([n_heads]); both start at zero.
    params: size, n_heads, dim, v_dim, gate_cap, eps."""

    @classmethod
    def declare_weights(cls, params):
        E, H, D, V = (params[k] for k in ("size", "n_heads", "dim", "v_dim"))
        return {"q_weight": WeightDecl((H * D, E), "matrix"), "k_weight": WeightDecl((H * D, E), "matrix"),
                "v_weight": WeightDecl((H * V, E), "matrix"), "gate_weight": WeightDecl((H * V, E), "matrix"),
                "in_gate_weight": WeightDecl((H, E), "matrix"), "in_gate_bias": WeightDecl((H,), "bias"),
                "forget_weight": WeightDecl((H, E), "matrix"), "forget_bias": WeightDecl((H,), "bias"),
                "norm": WeightDecl((H * V,), "norm_gain"), "out_weight": WeightDecl((E, H * V), "residual_matrix")}

    def load(self, tensors, store):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        refs = [tensors[k] for k in ("q_weight", "k_weight", "v_weight", "gate_weight", "in_gate_weight", "forget_weight")]
        n = 2 * H * D + 2 * H * V + 2 * H
        pad = (-n) % 8
        self.inp_w = store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0))
        bi, bf = tensors["in_gate_bias"], tensors["forget_bias"]
        bias = store.computed(f"0+{bi.name}+{bf.name}+{pad}", kind="vector", make=lambda: torch.cat(
            [torch.zeros(n - 2 * H), bi.tensor.float(), bf.tensor.float(), torch.zeros(pad)]))
        self.inp = Linear(self.inp_w, bias)
        self.norm = store.vector(tensors["norm"])
        self.out = Linear(store.matrix(tensors["out_weight"]), None)

    def cache_need(self):
        p = self.params
        return (CacheNeed.state((p["n_heads"], p["dim"], p["v_dim"] + 1), "float32"),
                CacheNeed.state((p["n_heads"],), "float32"))

    def workspace_per_token(self):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        return 4 * (2 * H * D + 2 * H * V + 2 * H + 8) + 12 * H + 4 * H * (V + 1) + act * H * V + 2048

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, D, V = p["n_heads"], p["dim"], p["v_dim"]
        T = h.shape[0]
        state, maxima = cache
        pre = ctx.alloc((T, self.inp.out_size), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        c_v, c_g, c_i = 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V
        gates = ctx.alloc((T, 2 * H), torch.float32)
        m_run = ctx.alloc((T, H), torch.float32)
        ops.stabilized_gates(ctx.columns(pre, c_i, c_i + H), ctx.columns(pre, c_i + H, c_i + 2 * H), float(p["gate_cap"]),
                             gates, m_run, maxima.tensor, ctx.q_start, ctx.state_slots, ctx.R, H)
        o = ctx.alloc((T, H * (V + 1)), torch.float32)
        ops.matrix_state("gated", ctx.columns(pre, 0, H * D), ctx.columns(pre, H * D, 2 * H * D),
                         ctx.columns(pre, c_v, c_g), o, state.tensor, ctx.q_start, ctx.state_slots, ctx.R, H, H, D, V + 1,
                         gates=gates, q_scale=float(D) ** -0.5, ones_col=True)
        y = ctx.alloc((T, H * V), self.rt.act_dtype)
        ops.gated_norm(o, ctx.columns(pre, c_g, c_i), self.norm, y, H, V, float(p["eps"]), "sigmoid", o_pitch=V + 1,
                       m_run=m_run)
        return self.out.forward(ctx, y, out=out, residual=residual)
