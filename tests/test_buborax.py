"""Buborax without a device: configuration, plan (the running order of a repeated run of layers),
tensors, cache groups per pass, pages given back behind a window, and the plain implementation's
own consistency."""
import copy

import numpy as np
import pytest

import plain_buborax as P
from buborax_models import BUB, make_dir, make_sharp_dir


def _cfg(name):
    from sglang_c_b200.config import resolve_architecture
    arch = resolve_architecture(BUB[name])
    return arch, arch.config_class.from_dict(BUB[name])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_config_round_trip_plan_and_tensors(name):
    from sglang_c_b200.weights.loader import required_tensors
    arch, cfg = _cfg(name)
    assert arch.name == "Buborax"
    assert arch.config_class.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == BUB[name]["layers"]
    plan = arch.build_plan(cfg)
    need = required_tensors(plan)
    d = BUB[name]
    E, layers = d["width"], d["layers"]
    # the running order is the plain implementation's
    want = P.layer_order(d)
    assert [(c.layer, None if c.enter is None else c.enter[1]) for c in plan.order] == want
    assert all(c.cache_of is None for c in plan.order)
    if "loop" in d:
        assert need["loop.in"].shape == (E, 2 * E) and need["loop.step"].shape == (d["loop"]["times"], E)
    else:
        assert "loop.in" not in need and plan.entries == []
    for i, layer in enumerate(layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            assert need[f"l{i}.mix.k"].shape == (m["kv_heads"] * m["dim"], E)
            assert need[f"l{i}.mix.talk"].shape == (m["heads"], m["heads"])
            assert need[f"l{i}.mix.q.norm"].shape == need[f"l{i}.mix.k.norm"].shape == (m["dim"],)
            assert need[f"l{i}.mix.g"].shape == (m["heads"] * m["dim"], E) and f"l{i}.mix.v" not in need
        elif layer["type"] == "hgrn2":
            assert need[f"l{i}.mix.f"].shape == (m["heads"] * m["dim"], E)
            assert need[f"l{i}.mix.f.b"].shape == need[f"l{i}.mix.lower"].shape == (m["heads"] * m["dim"],)
            assert need[f"l{i}.mix.v"].shape == (m["heads"] * m["vdim"], E) and need[f"l{i}.mix.norm"].shape == (m["vdim"],)
        else:
            assert need[f"l{i}.mix.q"].shape == (m["heads"] * (m["dim"] + m["rot_dim"]), E)
            assert need[f"l{i}.mix.dkv"].shape == (m["kv_rank"] + m["rot_dim"], E)
            assert need[f"l{i}.mix.dkv.norm"].shape == (m["kv_rank"],)
            assert need[f"l{i}.mix.uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
            assert need[f"l{i}.mix.o"].shape == (E, m["heads"] * m["vdim"])
        assert (f"l{i}.mlp.gate" in need) == (layer["mlp"] is not None) == (f"l{i}.norm2" in need)
        assert f"l{i}.mlp.gate.b" not in need
    assert plan.head.weights["weight"] == "head" and plan.embedding.weights["table"] == "embed"


def test_config_errors_name_the_key():
    from sglang_c_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(BUB["A"])

    def broken(change):
        d = copy.deepcopy(BUB["A"])
        change(d)
        with pytest.raises(ConfigError) as e:
            arch.config_class.from_dict(d)
        return str(e.value)

    assert "type" in broken(lambda d: d["layers"][0].update(type="delta"))
    assert "kv_heads" in broken(lambda d: d["layers"][2]["mixer"].update(kv_heads=3))
    assert "vdim" in broken(lambda d: d["layers"][2]["mixer"].update(vdim=8))          # the values are the keys
    assert "dims" in broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10))   # more than the turned part
    assert "kv_rank" in broken(lambda d: d["layers"][0]["mixer"].pop("kv_rank"))
    assert "loop" in broken(lambda d: d["loop"].update(stop=9))
    assert "groups" in broken(lambda d: d["norm"].update(groups=3))                     # 64 is no multiple of 3
    assert "eps" in broken(lambda d: d["norm"].pop("eps"))
    assert "size" in broken(lambda d: d["layers"][2]["mixer"].update(mask={}))
    # what may be left out: the window, the repeated run, the multiplier
    d = copy.deepcopy(BUB["A"])
    d.pop("loop"), d.pop("residual_mult"), d["layers"][2]["mixer"].pop("mask")
    cfg = arch.config_class.from_dict(d)
    assert cfg.loop is None and cfg.residual_mult == 1.0 and cfg.layers[2].mixer.window is None


def test_every_pass_keeps_its_own_cache_and_windows_release_pages():
    """A layer that runs in four passes has four caches (or states); equal needs share a group, so a
    page id is valid in all of them; pages behind a window return to the pool."""
    from sglang_c_b200.cache import CacheManager
    from sglang_c_b200.engine.model import Model

    class _Rt:                      # parts only look at the precision while they are built
        dtype = "float32"
        device = None

    arch, cfg = _cfg("A")
    model = Model(arch.build_plan(cfg), _Rt())
    needs, cache_of = model.cache_needs()
    assert len(needs) == 12 and all(n is not None for n in needs)
    cm = CacheManager(needs, cache_of, page_size=16, n_pages=12, max_requests=2)
    loop_rec = [cm.binding(i) for i in (1, 3, 5, 7)]
    loop_att = [cm.binding(i) for i in (2, 4, 6, 8)]
    assert len({b.group for b in loop_rec}) == 1 and len({b.group for b in loop_att}) == 1
    g = cm.groups[loop_att[0].group]
    assert len(g.calls) == 4 and g.need.window == 37 and g.need.shared and g.need.n_kv_heads == 2
    assert cm.groups[loop_rec[0].group].need.state_shape == (4, 16, 24)
    lat = cm.groups[cm.binding(0).group].need
    assert lat.shared and lat.n_kv_heads == 1 and lat.head_dim == 40 + 8 and lat.window == 21
    assert cm.add_request("a") is not None and cm.extend("a", 60)
    gi = loop_att[0].group
    assert all(p >= 0 for p in cm.block_table(gi, "a"))
    assert cm.extend("a", 100)              # a query at 60 sees 24..60: the first page is gone
    assert [p >= 0 for p in cm.block_table(gi, "a")] == [False, True, True, True, True, True, True]
    assert [p >= 0 for p in cm.block_table(cm.binding(0).group, "a")][:2] == [False, False]
    none = cm.groups[cm.binding(9).group]
    assert none.need.window is None and all(p >= 0 for p in cm.block_table(cm.binding(9).group, "a"))
    cm.check()
    cm.free_request("a")
    assert cm.n_free_pages() == 12


def test_plain_mechanisms_agree_with_themselves(tmp_path):
    """The oracle's own consistency: a position's logits do not depend on what follows; the recurrence
    carried in two pieces is the recurrence in one; a window of the whole length is no window; mixing
    the heads with the identity leaves ordinary attention; turning by position p and q leaves dot
    products that depend on p - q only."""
    d = make_dir(tmp_path, "A")
    cfg, w = P.read_model_dir(d)
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], 60)]
    full = P.forward(cfg, w, toks)
    assert np.abs(P.forward(cfg, w, toks[:41]) - full[:41]).max() < 1e-9
    q, f, v = rng.standard_normal((30, 2, 5)), rng.random((30, 2, 5)), rng.standard_normal((30, 2, 3))
    o, S = P.row_gated_state(q, f, v)
    o1, S1 = P.row_gated_state(q[:11], f[:11], v[:11])
    o2, S2 = P.row_gated_state(q[11:], f[11:], v[11:], S1)
    assert np.abs(np.concatenate([o1, o2]) - o).max() < 1e-12 and np.abs(S2 - S).max() < 1e-12
    qq, kk = rng.standard_normal((20, 4, 6)), rng.standard_normal((20, 2, 6))
    g = np.ones(6)
    a = P.talking_heads(qq, kk, g, g, np.eye(4), 0.5, 20, 1e-6)
    b = P.talking_heads(qq, kk, g, g, np.eye(4), 0.5, None, 1e-6)
    assert np.abs(a - b).max() < 1e-12
    c = P.talking_heads(qq, kk, g, g, np.eye(4), 0.5, 5, 1e-6)
    assert np.abs(a[:5] - c[:5]).max() < 1e-12 and np.abs(a[5:] - c[5:]).max() > 1e-3
    x, y = rng.standard_normal((1, 8)), rng.standard_normal((1, 8))
    dot = lambda p, q_: float(P.rotate_pairs(x, np.array([p]), 6, 100.0)[0] @ P.rotate_pairs(y, np.array([q_]), 6, 100.0)[0])
    assert abs(dot(17.0, 5.0) - dot(112.0, 100.0)) < 1e-9 and abs(dot(17.0, 5.0) - dot(17.0, 6.0)) > 1e-3
    assert P.layer_order({"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]


def test_sharp_models_remember_far_tokens(tmp_path):
    """What the sharp variant is for: a token changed far back moves the last logits."""
    d = make_sharp_dir(tmp_path, "A")
    cfg, w = P.read_model_dir(d)
    rng = np.random.default_rng(4)
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], 150)]
    ref = P.forward(cfg, w, toks)
    toks2 = list(toks)
    toks2[3] = (toks2[3] + 1) % cfg["vocab"]
    moved = np.abs(P.forward(cfg, w, toks2)[-1] - ref[-1]).max()
    assert moved > 2e-3 * ref.std(), moved / ref.std()
