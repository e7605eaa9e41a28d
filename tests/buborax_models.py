"""Small Buborax configurations for the tests, random model folders for them, and "sharp" variants
whose constants and weights are changed so that a lost key, a window edge that is one token off or
a lost state shows in the logits."""
import copy
import json
import os

import numpy as np
import torch


def _att(heads, kv_heads, dim, scale, window, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _rec(heads, dim, vdim, ff=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, window, rot_dims, base, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# A: every kind of mixer; a repeated run that holds a recurrence and an attention (each pass keeps a
# state and a cache of its own); grouped key heads; windows that are no multiple of a page; a layer
# without a window and one without feed-forward; a rotation of part of the turned entries; a
# multiplier that is no power of two
BUB_A = {"architecture": "Buborax", "vocab": 300, "width": 64, "residual_mult": 0.7, "norm": {"eps": 1e-6, "groups": 2},
         "loop": {"start": 1, "stop": 3, "times": 4},
         "layers": [_lat(3, 16, 8, 24, 40, 0.2, 21, 6, 10000.0, 96), _rec(4, 16, 24, 80), _att(4, 2, 16, 0.25, 37, None),
                    _att(2, 1, 32, 0.18, None, 72), _rec(1, 40, 8, None), _lat(2, 24, 16, 16, 48, 0.15, None, 16, 500.0, 64)]}
# B: sizes the tensor-core products and the tensor-core prompt attention take (latent row of 128 and
# of 64); no repeated run; one norm group; multiplier one; windows of several pages
BUB_B = {"architecture": "Buborax", "vocab": 257, "width": 128, "residual_mult": 1.0, "norm": {"eps": 1e-5, "groups": 1},
         "layers": [_att(2, 2, 64, 0.125, 160, 256), _lat(4, 32, 16, 32, 112, 0.125, 150, 16, 20000.0, 144),
                    _rec(2, 64, 64, 128), _lat(2, 64, 16, 64, 48, 0.1, 70, 16, 10000.0, None), _rec(2, 128, 32, 120)]}
# C: sizes that no vector load and no tensor-core tile fits; every layer repeated; one head; a window
# of one page and a window of three tokens; five norm groups
BUB_C = {"architecture": "Buborax", "vocab": 101, "width": 50, "residual_mult": 1.3, "norm": {"eps": 1e-5, "groups": 5},
         "loop": {"start": 0, "stop": 3, "times": 2},
         "layers": [_rec(3, 7, 5, 33), _att(3, 3, 10, 0.4, 8, 70), _lat(1, 9, 6, 11, 13, 0.3, 3, 4, 100.0, 21)]}
BUB = {"A": BUB_A, "B": BUB_B, "C": BUB_C}
PAGE = {"A": 16, "B": 16, "C": 8}


def make_dir(tmp, name, store_dtype="float32", seed=None):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = BUB[name]
    arch = resolve_architecture(d)
    out = os.path.join(str(tmp), f"bub_{name}_{store_dtype}")
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        write_random_model(out, arch, arch.config_class.from_dict(d), seed if seed is not None else 900 + ord(name),
                           scheme="varied", store_dtype=store_dtype)
    return out


def make_sharp_dir(tmp, name, store_dtype="float32"):
    """The model `name` with attention scores several times as large (normalised queries and keys
    have a root mean square near one whatever the weights are, so the config's multiplier is what
    sharpens the softmax: a key lost, misplaced, read from a stale page or let in across a window's
    edge then moves the logits by far more than rounding) and the recurrences' lower bounds close to
    one (the state remembers hundreds of tokens)."""
    import plain_buborax
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    base = make_dir(tmp, name, "float32")
    out = os.path.join(str(tmp), f"bub_sharp_{name}_{store_dtype}")
    if os.path.exists(os.path.join(out, "model.safetensors")):
        return out
    cfg, w = plain_buborax.read_model_dir(base)
    cfg = copy.deepcopy(cfg)
    for entry in cfg["layers"]:
        if entry["type"] in ("attention", "latent_attention"):
            entry["mixer"]["scale"] *= 12.0
    rng = np.random.default_rng(78)
    tensors = {}
    for k, v in w.items():
        a = np.array(v, dtype=np.float32)
        if k.endswith(".mix.lower"):
            a = (0.985 + 0.0149 * rng.random(a.shape)).astype(np.float32)
        elif k.endswith(".mix.q") or k.endswith(".mix.dkv"):
            a = a * 6.0            # (latent attention has no query norm: larger projections sharpen it)
        t = torch.from_numpy(a)
        tensors[k] = t.to(torch.bfloat16) if (store_dtype == "bfloat16" and t.dim() >= 2) else t
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors, metadata={"format": "pt"})
    return out
