"""Lubavik as a plan of parts: a token table; layers that add the normed result of a sublayer that
reads the stream itself, x += norm1(mixer(x)), x += norm2(ff(x)) (norms with a gain stored around
zero), then a gated input from a second token table, x += rms_norm(P (gelu(G x) * e_layer[token]));
the mixer is a matrix memory with exponential gates and a running maximum, softmax attention with
a norm over the whole query and key projections, half-split rotation and a sink per head (a layer
may read the keys and values an earlier layer cached), or chunked softmax attention with biases,
per-head norms and neighbour-pair rotation beside a gated linear attention with a decay per key
channel; the feed-forward is dense under a squared relu, or a mixture of experts with softmax
routing, renormalised and scaled weights and an always-on shared expert; a final norm and a head.

Tensor names: `embed`, `side.embed`, `final.norm`, `head`, and for layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.side.gate|proj|norm`, `l<i>.mix.*` (mlstm: q, k, v, g, o, norm, i, i.b, f, f.b; attention: q,
k, v, q.norm, k.norm, sink, o; parallel: left.q|k|v|o with `.b` each, left.q.norm, left.k.norm,
right.q|k|v|g|o|norm|a1|a2|a2.b) and `l<i>.mlp.*` (dense: up, down; experts: router,
e<j>.gate|up|down, shared.gate|up|down).
"""
from ..config.lubavik import LubavikConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerCall, LayerPlan, ModelPlan, PartSpec


def _rotary(rot, pairing):
    if rot is None:
        return None
    return {"dims": rot.dims, "base": rot.base, "scaling": None, "pairing": pairing}


def _mlstm(cfg, m, p):
    return PartSpec("mlstm", {"size": cfg.width, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim,
                              "gate_cap": m.gate_cap, "eps": cfg.norm_eps},
                    {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "gate_weight": p + "g",
                     "in_gate_weight": p + "i", "in_gate_bias": p + "i.b", "forget_weight": p + "f",
                     "forget_bias": p + "f.b", "norm": p + "norm", "out_weight": p + "o"})


def _attention(cfg, m, p):
    own = m.kv_from is None
    params = {"size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
              "scale": m.scale, "rotary": _rotary(m.rot, "halves"), "qk_norm": "row_gain", "eps": cfg.norm_eps,
              "chunk": None, "window": None, "sink": True, "bias": False, "own_kv": own}
    w = {"q_weight": p + "q", "q_norm": p + "q.norm", "sink": p + "sink", "out_weight": p + "o"}
    if own:
        w.update({"k_weight": p + "k", "v_weight": p + "v", "k_norm": p + "k.norm"})
    return PartSpec("rotary_attention", params, w)


def _parallel(cfg, m, p):
    le, ri = m.left, m.right
    left = ("rotary_attention", {"size": cfg.width, "n_heads": le.heads, "n_kv_heads": le.kv_heads, "head_dim": le.dim,
                                 "v_dim": le.vdim, "scale": le.scale, "rotary": _rotary(le.rot, "neighbours"),
                                 "qk_norm": "head_gain", "eps": cfg.norm_eps, "chunk": le.chunk, "window": None,
                                 "sink": False, "bias": True, "own_kv": True, "out_mult": m.left_scale})
    right = ("gated_linear_attention", {"size": cfg.width, "n_heads": ri.heads, "dim": ri.dim, "v_dim": ri.vdim,
                                        "tau": ri.tau, "eps": cfg.norm_eps, "out_mult": m.right_scale})
    w = {}
    for role, name in (("q_weight", "q"), ("q_bias", "q.b"), ("k_weight", "k"), ("k_bias", "k.b"), ("v_weight", "v"),
                       ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("out_weight", "o"),
                       ("out_bias", "o.b")):
        w["left." + role] = p + "left." + name
    for role, name in (("q_weight", "q"), ("k_weight", "k"), ("v_weight", "v"), ("gate_weight", "g"),
                       ("out_weight", "o"), ("norm", "norm"), ("decay_down", "a1"), ("decay_up", "a2"),
                       ("decay_bias", "a2.b")):
        w["right." + role] = p + "right." + name
    return PartSpec("side_by_side", {"size": cfg.width, "eps": cfg.norm_eps, "combine": "sum", "left": left,
                                     "right": right}, w)


def _mlp(cfg, mlp, p):
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return PartSpec("mlp", {"size": cfg.width, "inner_size": mlp.ff, "activation": "relu2", "bias": False},
                        {"up_weight": p + "up", "down_weight": p + "down"})
    w = {"router": p + "router"}
    for e in range(mlp.experts):
        w.update({f"gate_{e}": f"{p}e{e}.gate", f"up_{e}": f"{p}e{e}.up", f"down_{e}": f"{p}e{e}.down"})
    if mlp.shared_ff is not None:
        w.update({"shared_gate": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down"})
    return PartSpec("routed_experts", {"size": cfg.width, "inner_size": mlp.ff, "n_experts": mlp.experts, "top": mlp.top,
                                       "score": "softmax", "renorm": True, "weight_scale": mlp.router_scale,
                                       "correction": False, "shared_inner_size": mlp.shared_ff}, w)


def build_plan(cfg: LubavikConfig) -> ModelPlan:
    E, L = cfg.width, len(cfg.layers)
    norm = lambda name: PartSpec("rms_norm", {"size": E, "eps": cfg.norm_eps, "one_plus": True}, {"weight": name})
    layers, order = [], []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        if lc.type == "mlstm":
            mixer = _mlstm(cfg, lc.mixer, p + "mix.")
        elif lc.type == "attention":
            mixer = _attention(cfg, lc.mixer, p + "mix.")
        else:
            mixer = _parallel(cfg, lc.mixer, p + "mix.")
        ffn = _mlp(cfg, lc.mlp, p + "mlp.")
        parts = {}
        if cfg.token_side_dim is not None:
            parts["side"] = ("stream_mix", PartSpec(
                "token_gated_input", {"size": E, "dim": cfg.token_side_dim, "index": i, "n_layers": L,
                                      "vocab_size": cfg.vocab, "eps": cfg.norm_eps},
                {"table": "side.embed", "gate_weight": p + "side.gate", "proj_weight": p + "side.proj",
                 "norm": p + "side.norm"}))
        layers.append(LayerPlan(name=f"l{i}", block=PartSpec("post_norm", {"last": i == L - 1}), mixer=mixer,
                                norm1=norm(p + "norm1"), ffn=ffn, norm2=norm(p + "norm2") if ffn is not None else None,
                                parts=parts))
        kv_from = lc.mixer.kv_from if lc.type == "attention" else None
        order.append(LayerCall(i, cache_of=kv_from))
    return ModelPlan(
        hidden_size=E, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "size": E}, {"table": "embed"}),
        position=PartSpec("none", {}, {}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "size": E}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id)


register_architecture("Lubavik", LubavikConfig, build_plan, model_types=("lubavik",))
