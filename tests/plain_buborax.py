"""A plain, slow restatement of the Buborax architecture in float64 numpy, one function per
mechanism, sharing nothing with the engine: the oracle of the tests.  It reads a model folder
with its own small safetensors reader; recurrences run token by token; there is no cache and
no batch.

Notation: x [n, E] is the residual stream of n consecutive tokens from position 0; W x is
written x @ W.T for matrices stored [out, in].
"""
import json
import math
import os
import struct

import numpy as np


# -- files ---------------------------------------------------------------------------------
def read_model_dir(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif meta["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        w[name] = a.astype(np.float64).reshape(meta["shape"])
    return cfg, w


# -- small functions -----------------------------------------------------------------------
def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * gain


def group_norm(x, gain, eps, groups):
    """The layers' norm: the row in `groups` equal consecutive parts, each divided by its own root
    mean square; the whole times the gain."""
    n, E = x.shape
    parts = x.reshape(n, groups, E // groups)
    parts = parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)
    return parts.reshape(n, E) * gain


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def window_mask(n, size):
    """visible[i, j]: 0 <= i - j < size (no size: the whole past)."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    d = i - j
    return (d >= 0) & (d < size if size else True)


def rotate_pairs(v, positions, dims, base):
    """Neighbouring pairs (2i, 2i+1) of the first `dims` entries of the last axis turned by
    position * base^(-2i/dims); v [n, ..., D]."""
    out = v.copy()
    for i in range(dims // 2):
        a = positions * base ** (-2.0 * i / dims)
        a = a.reshape((-1,) + (1,) * (v.ndim - 2))
        c, s = np.cos(a), np.sin(a)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


# -- mixers --------------------------------------------------------------------------------
def head_slopes(heads):
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def mask_size(m):
    return (m.get("mask") or {}).get("size")


def talking_heads(q, k, gain_q, gain_k, talk, scale, size, eps):
    """q [n, H, D], k [n, G, D] as projected -> [n, H, D]: per-head RMS norm of both, scores with a
    linear distance penalty per head, window, softmax, the heads' weights mixed by `talk`, applied
    to the keys as projected."""
    n, H, D = q.shape
    G = k.shape[1]
    qn, kn = rms_norm(q, gain_q, eps), rms_norm(k, gain_k, eps)
    vis = window_mask(n, size)
    dist = (np.arange(n)[:, None] - np.arange(n)[None, :]).astype(np.float64)
    slopes = head_slopes(H)
    P = np.zeros((H, n, n))
    for a in range(H):
        s = qn[:, a] @ kn[:, a // (H // G)].T * scale - slopes[a] * dist
        P[a] = softmax_rows(s, vis)
    Pm = np.einsum("hg,gij->hij", talk, P)
    o = np.zeros((n, H, D))
    for a in range(H):
        o[:, a] = Pm[a] @ k[:, a // (H // G)]
    return o


def talking_attention(h, w, p, m, eps):
    """Softmax attention whose values are the un-normed keys, with a linear distance penalty per
    head, a sliding window, the heads' weights mixed after the softmax, and a sigmoid output gate."""
    n = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(n, H, D)
    k = (h @ w[p + "k"].T).reshape(n, G, D)
    o = talking_heads(q, k, w[p + "q.norm"], w[p + "k.norm"], w[p + "talk"], m["scale"], mask_size(m), eps)
    o = o.reshape(n, H * D) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def row_gated_state(q, f, v, S=None):
    """q, f [n, H, D], v [n, H, V]: S <- diag(f_t) S + (1 - f_t) v_t^T, o_t = S^T q_t, token by
    token from S (zero if not given).  Returns (o [n, H, V], the last S [H, D, V])."""
    n, H, D = q.shape
    V = v.shape[2]
    S = np.zeros((H, D, V)) if S is None else S.copy()
    o = np.zeros((n, H, V))
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    return o, S


def hgrn2(h, w, p, m, eps):
    """A matrix state per head whose forget gate also says what is written:
    S <- diag(f) S + (1 - f) v^T, o = S^T q, token by token."""
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(n, H, D)
    v = (h @ w[p + "v"].T).reshape(n, H, V)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).reshape(n, H, D)
    o, _ = row_gated_state(q, f, v)
    o = rms_norm(o, w[p + "norm"], eps).reshape(n, H * V)
    return o @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are up-projections of one normed latent per position, plus
    one turned key part that all heads share."""
    n = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    pos = np.arange(n, dtype=np.float64)
    q = (h @ w[p + "q"].T).reshape(n, H, D + Rd)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, rot["dims"], rot["base"])
    low = h @ w[p + "dkv"].T
    c = rms_norm(low[:, :R], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(low[:, R:], pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(n, H, D)
    v = (c @ w[p + "uv"].T).reshape(n, H, V)
    vis = window_mask(n, mask_size(m))
    o = np.zeros((n, H, V))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        o[:, a] = softmax_rows(s, vis) @ v[:, a]
    return o.reshape(n, H * V) @ w[p + "o"].T


MIXERS = {"attention": talking_attention, "hgrn2": hgrn2, "latent_attention": latent_attention}


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# -- the model -----------------------------------------------------------------------------
def layer_order(cfg):
    """[(layer, pass number or None)]: the looped range `times` times in a row, the rest once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [n, vocab] of a whole sequence (and, if asked, the stream after every layer run)."""
    eps, groups, mult = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("residual_mult", 1.0)
    x = w["embed"][np.asarray(tokens)]
    x0 = x.copy()
    kept = []
    for i, enter in layer_order(cfg):
        if enter is not None:
            x = np.concatenate([x, x0], -1) @ w["loop.in"].T + w["loop.step"][enter]
        lc, p = cfg["layers"][i], f"l{i}."
        h = group_norm(x, w[p + "norm1"], eps, groups)
        x = x + mult * MIXERS[lc["type"]](h, w, p + "mix.", lc["mixer"], eps)
        if lc.get("mlp") is not None:
            h = group_norm(x, w[p + "norm2"], eps, groups)
            x = x + mult * feed_forward(h, w, p + "mlp.")
        if keep_layers:
            kept.append(x.copy())
    logits = group_norm(x, w["final.norm"], eps, groups) @ w["head"].T
    return (logits, np.stack(kept)) if keep_layers else logits


_dirs = {}


def forward_dir(model_dir, tokens):
    """Logits [n, vocab] of a whole sequence through the model of a folder (read once)."""
    if model_dir not in _dirs:
        _dirs[model_dir] = read_model_dir(model_dir)
    cfg, w = _dirs[model_dir]
    return forward(cfg, w, tokens)
