"""Lubavik without a device: configuration, plan, tensors, cache groups (a layer that reads another
layer's keys and values, a mixer that keeps two things), and the plain implementation's own
consistency."""
import copy

import numpy as np
import pytest

import plain_lubavik as P
from lubavik_models import LUB, make_dir


def _cfg(name):
    from sglang_c_b200.config import resolve_architecture
    arch = resolve_architecture(LUB[name])
    return arch, arch.config_class.from_dict(LUB[name])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_config_round_trip_and_plan(name):
    from sglang_c_b200.weights.loader import required_tensors
    arch, cfg = _cfg(name)
    assert arch.name == "Lubavik"
    assert arch.config_class.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == LUB[name]["layers"]
    assert cfg.to_dict().get("token_side") == LUB[name].get("token_side")
    plan = arch.build_plan(cfg)
    need = required_tensors(plan)
    layers = LUB[name]["layers"]
    E, side = LUB[name]["width"], LUB[name].get("token_side")
    assert len(plan.order) == len(plan.layers) == len(layers)
    assert ("side.embed" in need) == (side is not None)
    if side:
        assert need["side.embed"].shape == (LUB[name]["vocab"], len(layers) * side["dim"])
    for i, layer in enumerate(layers):
        m, mlp = layer["mixer"], layer["mlp"]
        assert plan.order[i].layer == i and plan.order[i].cache_of == m.get("kv_from")
        assert need[f"l{i}.norm1"].shape == (E,) and (f"l{i}.norm2" in need) == (mlp is not None)
        assert (f"l{i}.side.gate" in need) == (side is not None)
        if side:
            assert need[f"l{i}.side.gate"].shape == (side["dim"], E) and need[f"l{i}.side.proj"].shape == (E, side["dim"])
        if layer["type"] == "mlstm":
            assert need[f"l{i}.mix.q"].shape == (m["heads"] * m["dim"], E)
            assert need[f"l{i}.mix.norm"].shape == (m["heads"] * m["vdim"],)
            assert need[f"l{i}.mix.i"].shape == (m["heads"], E) and need[f"l{i}.mix.f.b"].shape == (m["heads"],)
        elif layer["type"] == "attention":
            assert need[f"l{i}.mix.q.norm"].shape == (m["heads"] * m["dim"],) and need[f"l{i}.mix.sink"].shape == (m["heads"],)
            assert need[f"l{i}.mix.o"].shape == (E, m["heads"] * m["vdim"])
            for t in ("k", "v", "k.norm"):
                assert (f"l{i}.mix.{t}" in need) == ("kv_from" not in m)
            assert f"l{i}.mix.q.b" not in need
        else:
            le, ri = m["left"], m["right"]
            assert need[f"l{i}.mix.left.v"].shape == (le["kv_heads"] * le["vdim"], E)
            assert need[f"l{i}.mix.left.k.b"].shape == (le["kv_heads"] * le["dim"],)
            assert need[f"l{i}.mix.left.q.norm"].shape == need[f"l{i}.mix.left.k.norm"].shape == (le["dim"],)
            assert need[f"l{i}.mix.right.norm"].shape == (ri["vdim"],) and f"l{i}.mix.left.sink" not in need
            assert need[f"l{i}.mix.right.a2"].shape[0] == ri["heads"] * ri["dim"] and need[f"l{i}.mix.right.a2"].shape[1] <= 0
        if mlp is not None and mlp["kind"] == "moe":
            n = mlp["router"]["experts"]
            assert need[f"l{i}.mlp.router"].shape == (n, E) and f"l{i}.mlp.correction" not in need
            assert need[f"l{i}.mlp.e{n - 1}.down"].shape == (E, mlp["expert"]["ff"]) and f"l{i}.mlp.e{n}.up" not in need
            assert (f"l{i}.mlp.shared.up" in need) == ("shared" in mlp)
        elif mlp is not None:
            assert need[f"l{i}.mlp.up"].shape == (mlp["ff"], E) and f"l{i}.mlp.gate" not in need
    assert plan.head.weights["weight"] == "head" and plan.embedding.weights["table"] == "embed"


def test_config_errors_name_the_key():
    from sglang_c_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(LUB["A"])

    def broken(change):
        d = copy.deepcopy(LUB["A"])
        change(d)
        with pytest.raises(ConfigError) as e:
            arch.config_class.from_dict(d)
        return str(e.value)

    assert "type" in broken(lambda d: d["layers"][0].update(type="delta"))
    assert "gate_cap" in broken(lambda d: d["layers"][0]["mixer"].pop("gate_cap"))
    assert "kv_heads" in broken(lambda d: d["layers"][1]["mixer"].update(kv_heads=3))
    assert "tau" in broken(lambda d: d["layers"][2]["mixer"]["right"].pop("tau"))
    assert "left_scale" in broken(lambda d: d["layers"][2]["mixer"].pop("left_scale"))
    assert "dims" in broken(lambda d: d["layers"][2]["mixer"]["left"]["rot"].update(dims=13))
    assert "kv_from" in broken(lambda d: d["layers"][3]["mixer"].update(kv_from=4))          # not earlier
    assert "kv_from" in broken(lambda d: d["layers"][3]["mixer"].update(kv_from=0))          # not an attention layer
    assert "layer 1" in broken(lambda d: d["layers"][3]["mixer"].update(vdim=8))             # other sizes than its source
    assert "router" in broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=9))
    assert "eps" in broken(lambda d: d["norm"].pop("eps"))
    assert "dim" in broken(lambda d: d["token_side"].pop("dim"))


def test_cache_groups_of_shared_keys_and_of_mixers_that_keep_two_things():
    from sglang_c_b200.cache import CacheManager
    from sglang_c_b200.engine.model import Model
    arch, cfg = _cfg("A")
    plan = arch.build_plan(cfg)

    class HostOnly:                     # parts are built without a device here: only their needs are asked
        dtype, device = "float32", None
    model = Model(plan, HostOnly())
    needs, cache_of = model.cache_needs()
    assert cache_of == [None, None, None, 1, None]
    assert isinstance(needs[0], tuple) and [n.kind for n in needs[0]] == ["state", "state"]
    assert needs[0][0].state_shape == (4, 16, 25) and needs[0][1].state_shape == (4,)      # the normaliser's column
    assert needs[1] == needs[3] and needs[1].kind == "paged_kv" and needs[1].v_dim == 16 and needs[1].chunk is None
    assert [n.kind for n in needs[2]] == ["paged_kv", "state"] and needs[2][0].chunk == 24
    cm = CacheManager(needs, cache_of, page_size=8, n_pages=10, max_requests=2)
    b1, b3 = cm.binding(1), cm.binding(3)
    assert b1.group == b3.group and b1.write and not b3.write
    # pages and slots come back and are used again
    assert cm.add_request("a") is not None and cm.extend("a", 61)
    assert cm.add_request("b") is not None and not cm.extend("b", 30)
    assert cm.add_request("c") is None
    cm.free_request("a")
    assert cm.extend("b", 30) and cm.add_request("c") is not None
    cm.check()


def test_plain_mechanisms_agree_with_themselves(tmp_path):
    """The oracle's own consistency: a position's logits do not depend on what follows it; a key
    outside the query's chunk does not matter, the one just inside does; the sink takes weight away;
    the routing weights sum to the scale; the matrix memory does not depend on where its running
    maximum starts as long as state and maximum go together."""
    d = make_dir(tmp_path, "A")
    cfg, w = P.read_model_dir(d)
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], 60)]
    full = P.forward(cfg, w, toks)
    assert np.abs(P.forward(cfg, w, toks[:31]) - full[:31]).max() < 1e-9
    n, H, G, D, V = 20, 4, 2, 8, 6
    q, k, v = rng.standard_normal((n, H, D)), rng.standard_normal((n, G, D)), rng.standard_normal((n, G, V))
    base = P.softmax_attention(q, k, v, 0.7, chunk=8)
    k2 = k.copy(); k2[7] += 5.0
    assert np.array_equal(P.softmax_attention(q, k2, v, 0.7, chunk=8)[8:], base[8:])
    k2 = k.copy(); k2[8] += 5.0
    assert np.abs(P.softmax_attention(q, k2, v, 0.7, chunk=8)[9] - base[9]).max() > 1e-3
    sunk = P.softmax_attention(q, k, v, 0.7, sinks=np.full(H, 2.0))
    plain = P.softmax_attention(q, k, v, 0.7)
    assert (np.abs(sunk[0]) < np.abs(plain[0])).all()          # one key: its weight is below one
    dense = P.route(rng.standard_normal((30, 9)), 4, 2.5)
    assert np.allclose(dense.sum(-1), 2.5) and ((dense > 0).sum(-1) == 4).all()
    qq, kk, vv = rng.standard_normal((n, 2, D)), rng.standard_normal((n, 2, D)), rng.standard_normal((n, 2, V))
    ig, fg = rng.standard_normal((n, 2)) * 3, -np.abs(rng.standard_normal((n, 2)))
    o = P.mlstm_recurrence(qq, kk, vv, ig, fg)
    # without any stabiliser: S = sum of exp(cumulated gates) k v^T, divided by max(|n.q|, 1) + 1e-6 exp(m)
    for t in (0, 5, n - 1):
        F = np.cumsum(fg[:t + 1], 0)
        wgt = np.exp(ig[:t + 1] + F[-1] - F)                     # [t+1, heads]
        S = np.einsum("th,thd,thv->hdv", wgt, kk[:t + 1], vv[:t + 1])
        nn = np.einsum("th,thd->hd", wgt, kk[:t + 1])
        m = np.zeros(2)
        for s in range(t + 1):
            m = np.maximum(fg[s] + m, ig[s])
        den = np.maximum(np.abs((nn * qq[t]).sum(-1)), 1.0) + 1e-6 * np.exp(m)
        assert np.allclose(np.einsum("hdv,hd->hv", S, qq[t]) / den[:, None], o[t], rtol=1e-9, atol=1e-12)
