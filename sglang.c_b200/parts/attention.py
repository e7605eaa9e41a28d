"""Attention mixers."""
import torch

from ..cache.needs import CacheNeed
from .base import Part
from .linear import Linear, declare_linear
from .plan import WeightDecl
from .position import PositionEncoding
from .registry import register_part


@register_part("mixer", "causal_attention")
class CausalAttention(Part):
    """Causal multi-head attention over a paged cache:
    qkv = h·W + b, split q|k|v along the last axis, heads side by side; new keys
    and values go to the cache; each query attends to the keys at positions up to
    its own (within `window` if set); the heads' outputs, side by side, go
    through the output projection into the residual
    (reference src/gpt2.c:222-278).
    params: size, n_heads, n_kv_heads, head_dim, scale (the multiplier of q·k),
    window (None or a count of keys), bias, weight_layout."""

    @classmethod
    def declare_weights(cls, params):
        lay, bias = params.get("weight_layout", "linear"), params.get("bias", True)
        qkv_out = (params["n_heads"] + 2 * params["n_kv_heads"]) * params["head_dim"]
        qkv = declare_linear(params["size"], qkv_out, lay, bias)
        out = declare_linear(params["n_heads"] * params["head_dim"], params["size"], lay, bias,
                             init="residual_matrix")
        d = {"qkv_" + k: v for k, v in qkv.items()}
        d.update({"out_" + k: v for k, v in out.items()})
        return d

    def load(self, tensors, store):
        lay = self.params.get("weight_layout", "linear")
        self.qkv = Linear.from_refs(store, tensors["qkv_weight"], tensors.get("qkv_bias"), lay)
        self.out = Linear.from_refs(store, tensors["out_weight"], tensors.get("out_bias"), lay)

    def cache_need(self):
        p = self.params
        return CacheNeed.paged_kv(p["n_kv_heads"], p["head_dim"], p.get("window"))

    def workspace_per_token(self):
        p = self.params
        return (4 if self.rt.dtype == "float32" else 2) * (2 * p["n_heads"] + 2 * p["n_kv_heads"]) * p["head_dim"]

    def graph_bound(self, ctx):
        # A step of single tokens in few (token, head) items goes to the decode attention that
        # stages a block's whole key range in shared memory sized by the bound, and what a block
        # holds of an SM decides whether it can start, and prefetch, while the kernels ahead still
        # run: there the bound moves in steps of 128 keys up to 1024 and of about an eighth of the
        # length beyond (a capture every 128 steps costs less than the tighter bound wins).
        from ..csrc import ops
        if ctx.n_decode == ctx.T and ctx.T * self.params["n_heads"] < ops.STREAM_MIN_ITEMS:
            g = 128
            while g * 8 < ctx.max_keys:
                g *= 2
            return ((ctx.max_keys + g - 1) // g) * g
        return None

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        p = self.params
        H, Hkv, D = p["n_heads"], p["n_kv_heads"], p["head_dim"]
        T = h.shape[0]
        qkv = ctx.alloc((T, (H + 2 * Hkv) * D), self.rt.act_dtype)
        grp = ctx.group(cache.group)
        # a position part that acts inside the mixer turns the keys before they are cached: then
        # the projection cannot write them; one that leaves PositionEncoding.rotate as it is does not
        turns = position is not None and getattr(type(position), "rotate", None) is not PositionEncoding.rotate
        if turns:
            self.qkv.forward(ctx, h, out=qkv)
            kv_written = False
        else:
            kv_written = ctx.rt.project_qkv(ctx, h, self.qkv, qkv, cache, grp, H, Hkv, D)
        q = ctx.columns(qkv, 0, H * D)
        k = ctx.columns(qkv, H * D, (H + Hkv) * D)
        v = ctx.columns(qkv, (H + Hkv) * D, (H + 2 * Hkv) * D)
        if position is not None:
            position.rotate(ctx, q, k)
        o = ctx.alloc((T, H * D), self.rt.act_dtype)
        ctx.rt.attend(ctx, q, k, v, cache, grp, o, H, Hkv, D, float(p["scale"]), p.get("window"),
                      kv_written=kv_written)
        return self.out.forward(ctx, o, out=out, residual=residual)


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """Causal multi-head attention whose keys and values are made from one cached latent:
    c = rms_norm(h·Wdkvᵀ) (kv_rank wide, the only thing kept per position);
    head i: k = Wuk_i c, v = Wuv_i c, score = (q_i · k) * scale, ordinary softmax over the
    positions up to the query's own; out = Wo · [heads' results side by side].
    Queries are h·Wqᵀ, or, with `q_rank`, go through a latent of their own:
    q = Wuq · rms_norm(h·Wdqᵀ).  No position enters.  With `own_latent` false the layer has no
    Wdkv: it reads the latents another call cached (the plan's `cache_of`) through its own Wuk, Wuv.

    Computed in the absorbed form: q_i · (Wuk_i c) = (Wuk_iᵀ q_i) · c and
    sum_j p_j Wuv_i c_j = Wuv_i (sum_j p_j c_j), so attention runs on the latent itself as one
    shared key/value head of size kv_rank, and Wuk_iᵀ is folded into the query projection, Wuv_i
    into the output projection, once at load (in 64-bit, then rounded to the runtime's matrix
    precision).

    With `rot_dim` > 0 every query head has rot_dim more entries behind its qk_dim, and Wdkv has
    rot_dim more rows behind the latent's: one key part that all heads share and no norm touches.
    Both are turned by a rotary position part built from `rotary` (its params) and their dot product
    joins the score: score = (q_i . Wuk_i c + q_i_turned . k_turned) * scale.  The cache row is then
    [c | k_turned], the absorbed query [Wuk_i^T q_i | q_i_turned]; a head's weighted sum of rows
    carries rot_dim entries that the folded output matrix meets with zero columns.
    `out_mult`: a multiplier of the mixer's result, folded into the output matrix.
    params: size, n_heads, qk_dim, v_dim, kv_rank, q_rank (None or a size), scale,
    eps (of the latents' norms), own_latent, window, rot_dim (default 0), rotary (dims, base,
    pairing, scaling), out_mult (default 1)."""

    @classmethod
    def declare_weights(cls, params):
        E, H, D, V, R = params["size"], params["n_heads"], params["qk_dim"], params["v_dim"], params["kv_rank"]
        Rd = int(params.get("rot_dim") or 0)
        d = {"k_up": WeightDecl((H * D, R), "matrix"), "v_up": WeightDecl((H * V, R), "matrix"),
             "out_weight": WeightDecl((E, H * V), "residual_matrix")}
        if params.get("q_rank"):
            Q = params["q_rank"]
            d.update({"q_down": WeightDecl((Q, E), "matrix"), "q_norm": WeightDecl((Q,), "norm_gain"),
                      "q_up": WeightDecl((H * (D + Rd), Q), "matrix")})
        else:
            d["q_weight"] = WeightDecl((H * (D + Rd), E), "matrix")
        if params.get("own_latent", True):
            d.update({"kv_down": WeightDecl((R + Rd, E), "matrix"), "kv_norm": WeightDecl((R,), "norm_gain")})
        return d

    def load(self, tensors, store):
        p = self.params
        H, D, V, R, Q = p["n_heads"], p["qk_dim"], p["v_dim"], p["kv_rank"], p.get("q_rank")
        Rd = self.rot_dim = int(p.get("rot_dim") or 0)
        m = float(p.get("out_mult", 1.0))
        k_up, v_up, w_o = tensors["k_up"], tensors["v_up"], tensors["out_weight"]
        q_src = tensors["q_up"] if Q else tensors["q_weight"]

        def fold_queries():       # [H*(R+Rd), in]: head i's rows are Wuk_iᵀ · (head i's plain rows of the query
            uk = k_up.tensor.double().view(H, D, R)                      # projection), then its turned rows as they are
            wq = q_src.tensor.double().view(H, D + Rd, -1)
            folded = torch.einsum("hdr,hdi->hri", uk, wq[:, :D])
            return torch.cat([folded, wq[:, D:]], 1).reshape(H * (R + Rd), -1)

        def fold_output():        # [E, H*(R+Rd)]: head i's columns are (head i's columns of Wo) · Wuv_i, then zeros
            uv = v_up.tensor.double().view(H, V, R)
            wo = w_o.tensor.double().view(-1, H, V)
            folded = torch.einsum("ehv,hvr->ehr", wo, uv) * m
            return torch.cat([folded, folded.new_zeros(folded.shape[0], H, Rd)], 2).reshape(-1, H * (R + Rd))

        tag = (f",{Rd}" if Rd else "") + (f",*{m!r}" if m != 1.0 else "")
        # with a turned part the queries leave their product in 32-bit as well (the turn is 32-bit):
        # direct queries and the latent's projection, which read the same rows, are then one product
        self.q_abs = self.q_and_down = None
        if Rd and not Q and p.get("own_latent", True):
            kv = tensors["kv_down"]
            self.q_and_down = Linear(store.computed(
                f"fold({k_up.name},{q_src.name}{tag})+{kv.name}",
                lambda: torch.cat([fold_queries(), kv.tensor.double()], 0)), None)
        else:
            self.q_abs = Linear(store.computed(f"fold({k_up.name},{q_src.name}{tag})", fold_queries), None)
        self.out = Linear(store.computed(f"fold({w_o.name},{v_up.name}{tag})", fold_output), None)
        self.rotary = None
        if Rd:
            from .registry import get_part
            rot = dict(p.get("rotary") or {"dims": 0, "base": 10000.0})
            if int(rot.get("dims", 0)) > Rd:
                raise ValueError(f"latent attention: {rot['dims']} turned entries do not fit a turned part of {Rd}")
            self.rotary = get_part("position", "rotary")(rot, self.rt)
            self.rotary.load({}, store)
        self.q_norm = self.kv_norm = None
        downs = []
        if Q:
            downs.append(tensors["q_down"])
            self.q_norm = store.vector(tensors["q_norm"])
        if p.get("own_latent", True):
            downs.append(tensors["kv_down"])
            self.kv_norm = store.vector(tensors["kv_norm"])
        # the projections whose results go through a norm are one product with a 32-bit result
        self.down = None
        if downs and self.q_and_down is None:
            self.down = Linear(store.computed("+".join(r.name for r in downs),
                                              lambda: torch.cat([r.tensor.float() for r in downs], 0)), None)

    def cache_need(self):
        p = self.params
        return CacheNeed.paged_kv(1, p["kv_rank"] + int(p.get("rot_dim") or 0), p.get("window"), shared=True)

    def workspace_per_token(self):
        p = self.params
        act = 4 if self.rt.dtype == "float32" else 2
        W, Q = p["kv_rank"] + int(p.get("rot_dim") or 0), p.get("q_rank") or 0
        turned = 4 * (p["n_heads"] + 1) * W + 1024 if p.get("rot_dim") else 0
        return act * (2 * p["n_heads"] * W + Q) + 4 * (Q + W) + turned

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        from ..csrc import ops
        p = self.params
        H, R, Q = p["n_heads"], p["kv_rank"], p.get("q_rank") or 0
        own = p.get("own_latent", True)
        if own != cache.write:
            raise ValueError("latent attention: a layer with its own latent projection owns its cache, one without reads another's")
        T = h.shape[0]
        eps = float(p["eps"])
        grp = ctx.group(cache.group)
        if self.rot_dim:
            return self._forward_turned(ctx, h, residual, cache, grp, out)
        q_in = h
        if self.down is not None:
            low = ctx.alloc((T, self.down.out_size), torch.float32)
            self.down.forward(ctx, h, out=low)
            if Q:
                q_in = ctx.alloc((T, Q), self.rt.act_dtype)
                ops.norm_rows(ctx.columns(low, 0, Q), self.q_norm, None, eps, q_in, form="rms")
            if own:
                # the normalised latent goes straight into its cache rows (page * page_size + offset)
                rows = cache.tensor.view(-1, R)
                ops.norm_rows(ctx.columns(low, Q, Q + R), self.kv_norm, None, eps, rows, form="rms", dst_rows=grp.slots)
        q = ctx.alloc((T, H * R), self.rt.act_dtype)
        self.q_abs.forward(ctx, q_in, out=q)
        o = ctx.alloc((T, H * R), self.rt.act_dtype)
        ctx.rt.attend_shared(ctx, q, cache, grp, o, H, R, float(p["scale"]), p.get("window"))
        return self.out.forward(ctx, o, out=out, residual=residual)

    def _forward_turned(self, ctx, h, residual, cache, grp, out):
        """The form with a turned part: queries and the latent's row leave their products in 32-bit;
        one launch norms the latent, turns the shared key part and every head's turned entries, and
        writes the row into the cache and the queries in the activation precision."""
        from ..csrc import ops
        p = self.params
        H, R, Rd, Q = p["n_heads"], p["kv_rank"], self.rot_dim, p.get("q_rank") or 0
        own = p.get("own_latent", True)
        T, W = h.shape[0], R + Rd
        eps = float(p["eps"])
        low = None
        if self.q_and_down is not None:
            pre = ctx.alloc((T, H * W + W), torch.float32)
            self.q_and_down.forward(ctx, h, out=pre)
            qx, low = ctx.columns(pre, 0, H * W), ctx.columns(pre, H * W, H * W + W)
        else:
            q_in = h
            if self.down is not None:
                lows = ctx.alloc((T, self.down.out_size), torch.float32)
                self.down.forward(ctx, h, out=lows)
                if Q:
                    q_in = ctx.alloc((T, Q), self.rt.act_dtype)
                    ops.norm_rows(ctx.columns(lows, 0, Q), self.q_norm, None, eps, q_in, form="rms")
                if own:
                    low = ctx.columns(lows, Q, Q + W)
            qx = ctx.alloc((T, H * W), torch.float32)
            self.q_abs.forward(ctx, q_in, out=qx)
        q = ctx.alloc((T, H * W), self.rt.act_dtype)
        rot = self.rotary
        ops.latent_rope(qx, low, self.kv_norm, eps, ctx.positions, rot.frequencies, rot.multiplier, rot.dims,
                        rot.pairing, q, cache.tensor.view(-1, W) if own else None, grp.slots, H, R, Rd)
        o = ctx.alloc((T, H * W), self.rt.act_dtype)
        ctx.rt.attend_shared(ctx, q, cache, grp, o, H, W, float(p["scale"]), p.get("window"))
        return self.out.forward(ctx, o, out=out, residual=residual)


@register_part("mixer", "talking_attention")
class TalkingHeadsAttention(Part):
    """Softmax attention whose heads exchange their weights after the softmax, with grouped key
    heads that are also the values:
        q = h Wq^T, k = h Wk^T (n_kv_heads x head_dim), v = k as projected;
        q^, k^: each head divided by its root mean square (eps) times a gain of head_dim entries
        (one for the queries, one for the keys; the heads share them);
        s_a(i, j) = (q^_a(i) . k^_c(j)) * scale - slope_a (i - j),  c = a / (n_heads / n_kv_heads),
        slope_a = 2^(-slope_span (a + 1) / n_heads), over 0 <= i - j < window (all j <= i without);
        p_a = softmax_j s_a;   p'_a = sum_b talk[a][b] p_b;   o_a(i) = sum_j p'_a(i, j) v_c(j);
        result = Wo (o * sigmoid(h Wg^T)) * out_mult.
    The three input projections are one product with a 32-bit result; the cache keeps one row per
    position and key head, the key as projected (its 1/rms is formed where it is read).  Norms,
    scores, weights, their mix and the gate are 32-bit.
    params: size, n_heads, n_kv_heads, head_dim, scale, window, eps, slope_span (default 8),
    out_mult (default 1)."""

    @classmethod
    def declare_weights(cls, params):
        E, H, G, D = (params[k] for k in ("size", "n_heads", "n_kv_heads", "head_dim"))
        return {"q_weight": WeightDecl((H * D, E), "matrix"), "k_weight": WeightDecl((G * D, E), "matrix"),
                "q_norm": WeightDecl((D,), "norm_gain"), "k_norm": WeightDecl((D,), "norm_gain"),
                "talk": WeightDecl((H, H), "mixing"), "gate_weight": WeightDecl((H * D, E), "matrix"),
                "out_weight": WeightDecl((E, H * D), "residual_matrix")}

    def load(self, tensors, store):
        p = self.params
        H = p["n_heads"]
        refs = [tensors[k] for k in ("q_weight", "k_weight", "gate_weight")]
        pad = (-sum(r.tensor.shape[0] for r in refs)) % 8
        self.inp = Linear(store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0)), None)
        self.q_norm, self.k_norm = store.vector(tensors["q_norm"]), store.vector(tensors["k_norm"])
        self.talk = store.vector(tensors["talk"])
        self.out = Linear(store.matrix(tensors["out_weight"]), None)
        span = float(p.get("slope_span", 8.0))
        slopes = torch.tensor([2.0 ** (-span * (a + 1) / H) for a in range(H)], dtype=torch.float64)
        self.slopes = slopes.to(torch.float32).to(self.rt.device)

    def cache_need(self):
        p = self.params
        return CacheNeed.paged_kv(p["n_kv_heads"], p["head_dim"], p.get("window"), shared=True)

    def workspace_per_token(self):
        p = self.params
        H, G, D = p["n_heads"], p["n_kv_heads"], p["head_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        return 4 * ((2 * H + G) * D + 8) + 4 * H * D + act * H * D + 1024

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        from ..csrc import ops
        p = self.params
        H, G, D = p["n_heads"], p["n_kv_heads"], p["head_dim"]
        T = h.shape[0]
        eps = float(p["eps"])
        grp = ctx.group(cache.group)
        pre = ctx.alloc((T, self.inp.out_size), torch.float32)
        self.inp.forward(ctx, h, out=pre)
        q = ctx.alloc((T, H * D), torch.float32)
        ops.talk_prep(pre, self.q_norm, self.k_norm, eps, q, cache.tensor, grp.slots, H, G, D, grp.page_size)
        o = ctx.alloc((T, H * D), self.rt.act_dtype)
        gate = ctx.columns(pre, (H + G) * D, (2 * H + G) * D)
        scale, mult = float(p["scale"]), float(p.get("out_mult", 1.0))
        # bfloat16: tiles of 16 queries of a request on the tensor cores (a single token is a tile
        # of one row); 32-bit, and sizes without a tiled form: a block a token
        if self.rt.dtype != "bfloat16" or not ops.talk_attention_tiles(
                q, cache.tensor, grp.block_table, ctx.q_start, ctx.kv_len, self.slopes, self.talk, gate, o, ctx.R,
                ctx.max_q_len, H, G, D, grp.page_size, scale, eps, mult, p.get("window"), max_keys=ctx.max_keys):
            ops.talk_attention(q, cache.tensor, grp.block_table, ctx.token_req, ctx.positions, self.slopes, self.talk,
                               gate, o, H, G, D, grp.page_size, scale, eps, mult, p.get("window"))
        return self.out.forward(ctx, o, out=out, residual=residual)


@register_part("mixer", "rotary_attention")
class RotaryAttention(Part):
    """Causal softmax attention with grouped key/value heads whose sizes are free: queries and
    keys of `head_dim`, values of `v_dim`.  q, k, v are projections of h without biases (one product
    with a 32-bit result); q and k are turned by a `rotary` position part built from `rotary`
    (its params), then, with `qk_norm`, each head is divided by its root mean square (eps inside
    the root, no gain); score = (q . k) * scale.  `chunk`: position i sees j <= i only if both lie
    in the same chunk of so many positions, counted from position 0.  `window`: the usual sliding
    window.  `sink`: a learned score per head that joins the softmax's denominator once (it has no
    key and no value and is not scaled).  Query head i reads key/value head i / (n_heads / n_kv_heads).
    The cache keeps turned, normalised keys and plain values, a page's keys ahead of its values.
    Other forms of `qk_norm`, both BEFORE the turn and with learned gains: "head_gain": each head
    divided by its root mean square times a gain of head_dim entries (`q_norm`, `k_norm`) that the
    heads share; "row_gain": all query heads of a token divided by one root mean square over their
    n_heads x head_dim entries times a gain of that size (`q_norm`), the key heads likewise
    (`k_norm`).  The rotary params may ask for the pairing "neighbours".  `bias`: the four
    projections have biases.  `own_kv` false: the layer has no key and value projections (nor
    `k_norm`) and reads what another call cached (the plan's `cache_of`).  `out_mult`: a multiplier
    of the mixer's result (the values are cached times it: the attention is linear in them).
    params: size, n_heads, n_kv_heads, head_dim, v_dim, scale, rotary (dims, base, scaling, pairing) or
    None, qk_norm, eps, chunk, window, sink, bias (default false), own_kv (default true), out_mult
    (default 1)."""

    @classmethod
    def declare_weights(cls, params):
        E, H, G, D, V = (params[k] for k in ("size", "n_heads", "n_kv_heads", "head_dim", "v_dim"))
        own, bias, norm = params.get("own_kv", True), params.get("bias", False), params.get("qk_norm")
        d = {"q_weight": WeightDecl((H * D, E), "matrix"), "out_weight": WeightDecl((E, H * V), "residual_matrix")}
        if own:
            d.update({"k_weight": WeightDecl((G * D, E), "matrix"), "v_weight": WeightDecl((G * V, E), "matrix")})
        if bias:
            d.update({"q_bias": WeightDecl((H * D,), "bias"), "out_bias": WeightDecl((E,), "bias")})
            if own:
                d.update({"k_bias": WeightDecl((G * D,), "bias"), "v_bias": WeightDecl((G * V,), "bias")})
        if norm in ("head_gain", "row_gain"):
            d["q_norm"] = WeightDecl((D if norm == "head_gain" else H * D,), "norm_gain")
            if own:
                d["k_norm"] = WeightDecl((D if norm == "head_gain" else G * D,), "norm_gain")
        if params.get("sink"):
            d["sink"] = WeightDecl((H,), "bias")
        return d

    def load(self, tensors, store):
        from .registry import get_part
        p = self.params
        self.own = p.get("own_kv", True)
        self.mult = float(p.get("out_mult", 1.0))
        roles = ("q", "k", "v") if self.own else ("q",)
        refs = [tensors[k + "_weight"] for k in roles]
        n = sum(r.tensor.shape[0] for r in refs)
        pad = (-n) % 8
        bias = None
        if p.get("bias", False):
            brefs = [tensors[k + "_bias"] for k in roles]
            bias = store.computed("+".join(r.name for r in brefs) + f"+{pad}", kind="vector", make=lambda: torch.cat(
                [r.tensor.float() for r in brefs] + [torch.zeros(pad)]))
        self.qkv = Linear(store.computed("+".join(r.name for r in refs) + f"+{pad}", lambda: torch.cat(
            [r.tensor.float() for r in refs] + [torch.zeros(pad, refs[0].tensor.shape[1])], 0)), bias)
        out_bias = None
        if p.get("bias", False):
            ob, m = tensors["out_bias"], self.mult
            out_bias = store.vector(ob) if m == 1.0 else store.computed(
                f"{ob.name}*{m!r}", kind="vector", make=lambda: (ob.tensor.double() * m).float())
        self.out = Linear(store.matrix(tensors["out_weight"]), out_bias)
        self.sink = store.vector(tensors["sink"]) if p.get("sink") else None
        rot = p.get("rotary") or {"dims": 0, "base": 10000.0, "scaling": None}
        self.rotary = get_part("position", "rotary")(rot, self.rt)
        self.rotary.load({}, store)
        self.norm = p.get("qk_norm")
        self.q_gain = store.vector(tensors["q_norm"]) if "q_norm" in tensors else None
        self.k_gain = store.vector(tensors["k_norm"]) if "k_norm" in tensors else None
        # the first kernel of this mixer serves its first form: unit-RMS heads behind a turn of halves
        self.general = self.norm in ("head_gain", "row_gain") or self.rotary.pairing != "halves" or not self.own \
            or self.mult != 1.0

    def cache_need(self):
        p = self.params
        return CacheNeed.paged_kv(p["n_kv_heads"], p["head_dim"], p.get("window"), v_dim=p["v_dim"], chunk=p.get("chunk"))

    def workspace_per_token(self):
        p = self.params
        H, G, D, V = p["n_heads"], p["n_kv_heads"], p["head_dim"], p["v_dim"]
        act = 4 if self.rt.dtype == "float32" else 2
        from ..csrc import ops
        # (a step of single tokens deals a token's keys to several blocks: their shares)
        return 4 * ((H + G) * D + G * V + 8) + act * H * (D + V) + 1024 + 4 * H * ops.EXT_MAX_SPLITS * (V + 2)

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        from ..csrc import ops
        p = self.params
        H, G, D, V = p["n_heads"], p["n_kv_heads"], p["head_dim"], p["v_dim"]
        T = h.shape[0]
        grp = ctx.group(cache.group)
        if self.own != cache.write:
            raise ValueError("rotary_attention: a layer with key and value projections owns its cache, one "
                             "without reads another's")
        pre = ctx.alloc((T, self.qkv.out_size), torch.float32)
        self.qkv.forward(ctx, h, out=pre)
        q = ctx.alloc((T, H * D), self.rt.act_dtype)
        if self.general:
            Gown = G if self.own else 0
            ops.qk_prep(ctx.columns(pre, 0, H * D + Gown * (D + V)), ctx.positions, self.rotary.frequencies,
                        self.rotary.multiplier, self.rotary.dims, self.rotary.pairing, self.norm, float(p["eps"]),
                        self.q_gain, self.k_gain, q, cache.tensor if self.own else None,
                        grp.slots if self.own else None, H, Gown, D, V, grp.page_size, v_mult=self.mult)
        else:
            ops.rotary_kv(ctx.columns(pre, 0, (H + G) * D + G * V), ctx.positions, self.rotary.frequencies,
                          self.rotary.multiplier, self.rotary.dims, float(p["eps"]) if p.get("qk_norm") else None, q,
                          cache.tensor, grp.slots, H, G, D, V, grp.page_size)
        o = ctx.alloc((T, H * V), self.rt.act_dtype)
        # a step of prompt portions only, keys and values of one size the tensor-core kernel takes (a
        # page is then its [2][G][page_size][D]): 128-query tiles on the tensor cores; every other
        # step (single tokens among them, other sizes, 32-bit) goes to the general kernel
        if D == V and ctx.n_decode == 0 and ctx.max_q_len > 1 and self.rt.dtype == "bfloat16":
            pages = cache.tensor.view(cache.tensor.shape[0], 2, G, grp.page_size, D)
            if ops.attention_prefill_tc_supported(q, pages, float(p["scale"])) and o.stride(0) % 8 == 0:
                ops.attention_prefill_tc(q, pages, grp.block_table, ctx.q_start, ctx.kv_len, o, H, float(p["scale"]),
                                         p.get("window"), ctx.R, ctx.max_q_len, chunk=p.get("chunk"), sinks=self.sink)
                return self.out.forward(ctx, o, out=out, residual=residual)
        # every other step goes to the general kernel; where every request brings one token, a
        # token's keys are dealt to several blocks and a second launch merges their shares
        splits = ops.attention_ext_splits(ctx.max_keys, p.get("window"), p.get("chunk")) if ctx.max_q_len == 1 else 1
        ws = ctx.alloc((T * H * splits * (V + 2),), torch.float32) if splits > 1 else None
        ops.attention_ext(q, cache.tensor, grp.block_table, ctx.token_req, ctx.positions, o, H, G, D, V, grp.page_size,
                          float(p["scale"]), p.get("window"), p.get("chunk"), self.sink, ctx.max_keys,
                          max_q_len=ctx.max_q_len, splits=splits, workspace=ws)
        return self.out.forward(ctx, o, out=out, residual=residual)


@register_part("mixer", "side_by_side")
class SideBySideMixers(Part):
    """Two mixers that read the same rows; the result is half the sum of their outputs, each first
    RMS-normed over the model width with a gain of its own:
        mix(h) = (rms_norm(left(h)) * g_left + rms_norm(right(h)) * g_right) / 2.
    Each side keeps what it needs (the layer's cache need is the pair of theirs).  The halves are
    folded into the gains at load, and each side's norm adds straight into the 32-bit stream.
    With `combine` "sum" the result is the plain sum of the sides' results, mix(h) = left(h) +
    right(h), with no norms and no gains of its own (a side that is to count with a multiplier
    takes it as its own parameter): the left side's last product writes, the right side's adds.
    params: size, eps, left: (kind, params), right: (kind, params), combine ("normed_half_sum", the
    default, or "sum"); weights: the sides' own under `left.` / `right.`, and (first form only)
    `left_out`, `right_out`."""

    SIDES = ("left", "right")

    @classmethod
    def _side_class(cls, params, side):
        from .registry import get_part
        kind, sub = params[side]
        return get_part("mixer", kind), sub

    @classmethod
    def declare_weights(cls, params):
        d = {}
        for side in cls.SIDES:
            klass, sub = cls._side_class(params, side)
            d.update({f"{side}.{role}": decl for role, decl in klass.declare_weights(sub).items()})
            if params.get("combine", "normed_half_sum") != "sum":
                d[f"{side}_out"] = WeightDecl((params["size"],), "norm_gain")
        return d

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.sides = []
        for side in self.SIDES:
            klass, sub = self._side_class(params, side)
            self.sides.append(klass(sub, runtime))
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.sides)
        self.plain_sum = params.get("combine", "normed_half_sum") == "sum"
        if params.get("combine", "normed_half_sum") not in ("normed_half_sum", "sum"):
            raise ValueError(f"side_by_side: combine {params['combine']!r}; known: normed_half_sum, sum")

    def load(self, tensors, store):
        self.gains = []
        for side, part in zip(self.SIDES, self.sides):
            part.load({role[len(side) + 1:]: ref for role, ref in tensors.items() if role.startswith(side + ".")}, store)
            if self.plain_sum:
                continue
            ref = tensors[f"{side}_out"]
            self.gains.append(store.computed(ref.name + "/2", kind="vector", make=lambda r=ref: r.tensor.float() * 0.5))

    def cache_need(self):
        return tuple(m.cache_need() for m in self.sides)

    def workspace_per_token(self):
        return 4 * self.params["size"] + max(m.workspace_per_token() for m in self.sides)

    def graph_bound(self, ctx):
        asked = [b for b in (m.graph_bound(ctx) for m in self.sides) if b is not None]
        return max(asked) if asked else None

    def forward(self, ctx, h, residual, cache, position=None, out=None):
        from ..csrc import ops
        if self.plain_sum:
            # the left side writes its result, the right side's last product adds to it
            if out is None:
                for part, binding in zip(self.sides, cache):
                    mark = ctx.mark()
                    part.forward(ctx, h, residual=residual, cache=binding, position=position)
                    ctx.release(mark)
                return residual
            mark = ctx.mark()
            self.sides[0].forward(ctx, h, residual=None, cache=cache[0], position=position, out=out)
            ctx.release(mark)
            self.sides[1].forward(ctx, h, residual=out, cache=cache[1], position=position)
            ctx.release(mark)
            return out
        if out is not None:
            raise ValueError("side_by_side adds into the residual stream; it has no separate output")
        T, E = h.shape[0], self.params["size"]
        y = ctx.alloc((T, E), torch.float32)
        inner = ctx.mark()
        for part, binding, gain in zip(self.sides, cache, self.gains):
            part.forward(ctx, h, residual=None, cache=binding, position=position, out=y)
            ctx.release(inner)
            ops.norm_rows(y, gain, None, float(self.params["eps"]), residual[:T], form="rms", add=True)
        return residual
