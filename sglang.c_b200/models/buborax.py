"""Buborax as a plan of parts: a token table; pre-norm layers x += m mixer(norm1(x)),
x += m ff(norm2(x)) whose norms are RMS norms in groups; the mixer is a talking-heads attention
over un-normed keys that are also the values (distance penalty, window, output gate), an HGRN2
recurrence, or attention over a cached latent with a turned key part (neighbouring pairs, window);
the feed-forward is a gated MLP under the tanh form of GELU, without biases, or absent; a run of
layers may repeat with the same weights, each pass with a cache and state of its own and an input
re-entry ahead of it; a final grouped norm and a head of its own.  The multiplier m is taken by
each sublayer's stage ahead of its last product.

Tensor names: `embed`, `final.norm`, `head`, `loop.in`, `loop.step`, and for layer i
`l<i>.norm1|norm2`, `l<i>.mix.*` (attention: q, k, q.norm, k.norm, talk, g, o; hgrn2: q, f, f.b,
lower, v, norm, o; latent attention: q, dkv, dkv.norm, uk, uv, o) and `l<i>.mlp.gate|up|down`.
"""
from ..config.buborax import BuboraxConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerCall, LayerPlan, ModelPlan, PartSpec

SLOPE_SPAN = 8.0        # head a's distance penalty is 2^(-SLOPE_SPAN (a + 1) / heads) per position


def _mixer(cfg, lc, p):
    m, E, mult = lc.mixer, cfg.width, cfg.residual_mult
    if lc.type == "attention":
        return PartSpec("talking_attention",
                        {"size": E, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
                         "window": m.window, "eps": cfg.norm_eps, "slope_span": SLOPE_SPAN, "out_mult": mult},
                        {"q_weight": p + "q", "k_weight": p + "k", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
                         "talk": p + "talk", "gate_weight": p + "g", "out_weight": p + "o"})
    if lc.type == "hgrn2":
        return PartSpec("hgrn2", {"size": E, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim, "eps": cfg.norm_eps,
                                  "out_mult": mult},
                        {"q_weight": p + "q", "gate_weight": p + "f", "gate_bias": p + "f.b", "lower": p + "lower",
                         "v_weight": p + "v", "norm": p + "norm", "out_weight": p + "o"})
    return PartSpec("latent_attention",
                    {"size": E, "n_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim, "kv_rank": m.kv_rank,
                     "q_rank": None, "scale": m.scale, "eps": cfg.norm_eps, "own_latent": True, "window": m.window,
                     "rot_dim": m.rot_dim, "out_mult": mult,
                     "rotary": {"dims": m.rot_dims, "base": m.rot_base, "scaling": None, "pairing": "neighbours"}},
                    {"q_weight": p + "q", "kv_down": p + "dkv", "kv_norm": p + "dkv.norm", "k_up": p + "uk",
                     "v_up": p + "uv", "out_weight": p + "o"})


def build_plan(cfg: BuboraxConfig) -> ModelPlan:
    E = cfg.width
    norm = lambda name: PartSpec("rms_norm", {"size": E, "eps": cfg.norm_eps, "groups": cfg.norm_groups},
                                 {"weight": name})
    layers = []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = None
        if lc.ff is not None:
            ffn = PartSpec("gated_mlp", {"size": E, "inner_size": lc.ff, "bias": False, "activation": "gelu_tanh",
                                         "out_mult": cfg.residual_mult},
                           {"gate_weight": p + "mlp.gate", "up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
        layers.append(LayerPlan(name=f"l{i}", block=PartSpec("pre_norm"), norm1=norm(p + "norm1"),
                                mixer=_mixer(cfg, lc, p + "mix."),
                                norm2=norm(p + "norm2") if ffn is not None else None, ffn=ffn))
    # the running order: the repeated run of layers `times` times in a row, every call with a cache of
    # its own; the first call of each pass is preceded by the input re-entry with the pass's number
    entries, order = [], []
    n, lp = len(cfg.layers), cfg.loop
    if lp is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        entries.append(PartSpec("input_reentry", {"size": E, "times": lp.times},
                                {"in_weight": "loop.in", "steps": "loop.step"}))
        order = [LayerCall(i) for i in range(lp.start)]
        for t in range(lp.times):
            order += [LayerCall(i, enter=(0, t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        order += [LayerCall(i) for i in range(lp.stop, n)]
    return ModelPlan(
        hidden_size=E, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "size": E}, {"table": "embed"}),
        position=PartSpec("none", {}, {}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "size": E}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id, entries=entries)


register_architecture("Buborax", BuboraxConfig, build_plan, model_types=("buborax",))
