"""Small Lubavik configurations for the tests, random model folders for them, and "sharp" variants
whose constants and weights are changed so that a lost key, a chunk edge that is one token off, a
dropped sink or a lost state shows in the logits."""
import copy
import json
import os

import numpy as np
import torch


def _rot(base, dims):
    return {"base": base, "dims": dims}


def _mlstm(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def _attn(heads, kv_heads, dim, vdim, scale, rot=None, mlp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _left(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    return m


def _par(left, right, ls, rs, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def _right(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, scale, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


# A: every kind of layer and feed-forward; keys and values read from an earlier layer, with another
# layer in between; a chunk that is no multiple of a page; partial rotations of both pairings; a
# shared expert of another width than the routed ones; a layer without feed-forward; value sizes that
# differ from the key sizes
LUB_A = {"architecture": "Lubavik", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
         "layers": [
             _mlstm(4, 16, 24, 8.0, _dense(96)),
             _attn(4, 2, 32, 16, 0.2, _rot(10000.0, 16), _moe(8, 2, 40, 1.5, shared=24)),
             _par(_left(4, 2, 24, 16, 0.25, 24, _rot(5000.0, 12)), _right(2, 24, 40, 8.0), 0.7, 1.3, None),
             _attn(2, 2, 32, 16, 0.3, _rot(10000.0, 16), _dense(80), kv_from=1),
             _mlstm(1, 40, 8, 15.0, _moe(6, 3, 24, 1.0))]}
# B: sizes the tensor-core kernels take (head size 64 on both sides, equal key and value sizes, a
# chunk of several pages); one expert chosen; no token-side input; full rotations; no shared expert;
# an attention without rotation; a left side without a chunk mask
LUB_B = {"architecture": "Lubavik", "vocab": 257, "width": 72, "norm": {"eps": 1e-5},
         "layers": [
             _par(_left(2, 1, 64, 64, 0.125, 128, _rot(500000.0, 64)), _right(3, 64, 32, 4.0), 1.0, 1.0, _dense(144)),
             _attn(2, 1, 64, 64, 0.125, None, _moe(6, 1, 64, 2.0)),
             _mlstm(2, 128, 64, 10.0, _dense(80)),
             _par(_left(2, 2, 64, 64, 0.125, None, _rot(100.0, 32)), _right(1, 128, 16, 32.0), 0.5, 2.0,
                  _moe(4, 2, 32, 0.5, shared=32))]}
# C: sizes that no vector load and no tensor-core tile fits; all experts chosen; a chunk shorter than
# a page; one head; a token-side input of one entry; the first layer reads nobody's keys
LUB_C = {"architecture": "Lubavik", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "token_side": {"dim": 1},
         "layers": [
             _attn(3, 1, 10, 6, 0.4, _rot(100.0, 6), _moe(5, 5, 11, 3.0, shared=7)),
             _par(_left(3, 3, 10, 6, 0.4, 5, _rot(100.0, 10)), _right(1, 9, 3, 2.0), 0.9, 0.4, _dense(70)),
             _attn(6, 1, 10, 6, 0.2, _rot(100.0, 6), None, kv_from=0),
             _mlstm(3, 7, 5, 3.0, _dense(33))]}
LUB = {"A": LUB_A, "B": LUB_B, "C": LUB_C}
PAGE = {"A": 16, "B": 16, "C": 8}


def _rewrite(src, out, store_dtype, change, cfg_change=None):
    """The folder `src` (32-bit) written again as `out` with change(name, array) applied to every tensor."""
    import plain_lubavik
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    cfg, w = plain_lubavik.read_model_dir(src)
    cfg = copy.deepcopy(cfg)
    if cfg_change is not None:
        cfg_change(cfg)
    tensors = {}
    for k, v in w.items():
        t = torch.from_numpy(np.ascontiguousarray(change(k, np.array(v, dtype=np.float32)), dtype=np.float32))
        tensors[k] = t.to(torch.bfloat16) if (store_dtype == "bfloat16" and t.dim() >= 2) else t
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors, metadata={"format": "pt"})
    return out


def _lively(k, a):
    """Random weights of the usual small size leave two things degenerate here: a token table of
    entries around 0.02 puts the first layer's read-outs far below the eps of its norms, and router
    logits that are all alike make every choice a close call, which rounding decides.  So the token
    table is made of entries around one and the routers' rows are spread out."""
    if k == "embed":
        return a * 50.0
    if k.endswith(".mlp.router"):
        return a * 12.0
    return a


def make_dir(tmp, name, store_dtype="float32", seed=None):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = LUB[name]
    arch = resolve_architecture(d)
    out = os.path.join(str(tmp), f"lub_{name}_{store_dtype}")
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        raw = write_random_model(out + "_raw", arch, arch.config_class.from_dict(d),
                                 seed if seed is not None else 700 + ord(name), scheme="varied", store_dtype="float32")
        _rewrite(raw, out, store_dtype, _lively)
    return out


def make_sharp_dir(tmp, name, store_dtype="float32"):
    """The model `name` with attention scores several times as large (queries and keys are normed,
    so the config's multiplier is what sharpens the softmax: a key lost, misplaced, read from a stale
    page or let in across a chunk's edge then moves the logits by far more than rounding), sinks
    raised so that they carry weight, the linear attention's decays close to one (the decays' biases
    raised: the state remembers hundreds of tokens) and the matrix memory's forget gates close to one."""
    base = make_dir(tmp, name, "float32")
    out = os.path.join(str(tmp), f"lub_sharp_{name}_{store_dtype}")
    if os.path.exists(os.path.join(out, "model.safetensors")):
        return out

    def sharper(cfg):
        for entry in cfg["layers"]:
            if entry["type"] == "parallel":
                entry["mixer"]["left"]["scale"] *= 6.0
            elif entry["type"] == "attention":
                entry["mixer"]["scale"] *= 6.0

    def change(k, a):
        if k.endswith(".mix.right.a2.b"):
            return a + 5.0
        if k.endswith(".mix.f.b"):
            return a + 4.0
        if k.endswith(".mix.sink"):
            return a + 1.5
        return a

    return _rewrite(base, out, store_dtype, change, sharper)
