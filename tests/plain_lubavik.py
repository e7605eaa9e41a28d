"""A plain, slow restatement of the Lubavik architecture in float64 numpy, one function per
mechanism, sharing nothing with the engine: the oracle of the tests.  It reads a model folder
with its own small safetensors reader and runs whole sequences token by token where a
mechanism is a recurrence; there is no cache and no batch.

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


def log_sigmoid(v):
    return -(np.maximum(-v, 0.0) + np.log1p(np.exp(-np.abs(v))))


def silu(v):
    return v * sigmoid(v)


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))


def rms(x, eps):
    return np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """The model's norm: the weight is stored around zero."""
    return x / rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return x / rms(x, eps) * w


# -- rotations -----------------------------------------------------------------------------
def rotate(x, positions, dims, base, layout):
    """x [n, heads, D]: the first `dims` entries of every head turned by position * base^(-2i/dims);
    layout "neighbours" pairs entry 2i with 2i+1, "halves" pairs i with i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=np.float64) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * f[None, None, :]
    cs, sn = np.cos(a), np.sin(a)
    y = x.copy()
    if layout == "neighbours":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2] = u * cs - v * sn
        y[..., 1:dims:2] = v * cs + u * sn
    else:
        u, v = x[..., :half], x[..., half:dims]
        y[..., :half] = u * cs - v * sn
        y[..., half:dims] = v * cs + u * sn
    return y


# -- softmax attention ---------------------------------------------------------------------
def softmax_attention(q, k, v, scale, chunk=None, sinks=None):
    """q [n, H, D], k [n, G, D], v [n, G, V] at positions 0..n-1.  Query i sees j <= i, and with
    `chunk` only those j in its own chunk of so many positions.  `sinks` [H]: one more term
    exp(sink) in the denominator."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            lo = (i // chunk) * chunk if chunk else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sinks is None else max(s.max(), sinks[h])
            e = np.exp(s - m)
            den = e.sum() + (math.exp(sinks[h] - m) if sinks is not None else 0.0)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(0) / den
    return out


def attention_keys_values(w, p, m, h, positions, eps):
    """Keys (normed over the whole projection, turned) and values of an "attention" layer."""
    n = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = norm_plain(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(n, G, D)
    rot = m.get("rot")
    if rot:
        k = rotate(k, positions, rot["dims"], rot["base"], "halves")
    return k, (h @ w[p + "v"].T).reshape(n, G, V)


def attention_mixer(w, p, m, h, eps, kv):
    """kv = (keys, values) as the layer that owns them made them."""
    n = h.shape[0]
    H, D = m["heads"], m["dim"]
    pos = np.arange(n)
    q = norm_plain(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(n, H, D)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], "halves")
    o = softmax_attention(q, kv[0], kv[1], m["scale"], sinks=w[p + "sink"])
    return o.reshape(n, -1) @ w[p + "o"].T


# -- the side-by-side mixer ----------------------------------------------------------------
def left_side(w, p, m, h, eps):
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(n, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(n, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(n, G, V)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], "neighbours")
        k = rotate(k, pos, rot["dims"], rot["base"], "neighbours")
    mask = m.get("mask")
    o = softmax_attention(q, k, v, m["scale"], chunk=mask["size"] if mask else None)
    return o.reshape(n, -1) @ w[p + "o"].T + w[p + "o.b"]


def gated_linear_attention(q, k, v, alpha):
    """q, k, alpha [n, H, D], v [n, H, V]: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t."""
    n, H, D = q.shape
    S = np.zeros((H, D, v.shape[2]))
    out = np.zeros((n, H, v.shape[2]))
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def right_side(w, p, m, h, eps):
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(n, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(n, H, D)
    v = (h @ w[p + "v"].T).reshape(n, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = np.exp(log_sigmoid(z) / m["tau"]).reshape(n, H, D)
    o = gated_linear_attention(q, k, v, alpha)
    o = norm_plain(o, w[p + "norm"], eps).reshape(n, H * V)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(w, p, m, h, eps):
    return m["left_scale"] * left_side(w, p + "left.", m["left"], h, eps) \
        + m["right_scale"] * right_side(w, p + "right.", m["right"], h, eps)


# -- matrix memory -------------------------------------------------------------------------
def mlstm_recurrence(q, k, v, i_gate, f_gate):
    """q, k [n, H, D], v [n, H, V], log gates [n, H].  The running maximum starts at 0."""
    n, H, D = q.shape
    V = v.shape[2]
    S, nrm, mx = np.zeros((H, D, V)), np.zeros((H, D)), np.zeros(H)
    out = np.zeros((n, H, V))
    for t in range(n):
        m_new = np.maximum(f_gate[t] + mx, i_gate[t])
        keep, take = np.exp(f_gate[t] + mx - m_new), np.exp(i_gate[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        nrm = keep[:, None] * nrm + take[:, None] * k[t]
        mx = m_new
        den = np.maximum(np.abs((nrm * q[t]).sum(-1)), np.exp(-mx)) + 1e-6
        out[t] = np.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    return out


def mlstm_mixer(w, p, m, h, eps):
    n = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(n, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(n, H, D)
    v = (h @ w[p + "v"].T).reshape(n, H, V)
    i_gate = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f_gate = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = mlstm_recurrence(q, k, v, i_gate, f_gate)
    o = (o / rms(o, eps)).reshape(n, H * V) * w[p + "norm"]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# -- feed-forwards -------------------------------------------------------------------------
def dense_ff(w, p, h):
    return np.maximum(h @ w[p + "up"].T, 0.0) ** 2 @ w[p + "down"].T


def gated_expert(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(z, top, scale):
    """z [n, X] router logits -> dense weights [n, X]: softmax, the `top` largest kept, divided by
    their sum (+ 1e-20), times scale."""
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    dense = np.zeros_like(s)
    for t in range(s.shape[0]):
        chosen = np.argsort(-s[t], kind="stable")[:top]
        dense[t, chosen] = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * scale
    return dense


def moe_ff(w, p, mlp, h):
    r = mlp["router"]
    dense = route(h @ w[p + "router"].T, r["top"], r["scale"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for e in range(r["experts"]):
        rows = np.nonzero(dense[:, e])[0]
        if rows.size:
            out[rows] += dense[rows, e][:, None] * gated_expert(w, f"{p}e{e}.", h[rows])
    if mlp.get("shared"):
        out += gated_expert(w, p + "shared.", h)
    return out


# -- the per-layer token input -------------------------------------------------------------
def token_side(w, p, cfg, i, tokens, x):
    d = cfg["token_side"]["dim"]
    e = w["side.embed"][tokens][:, i * d:(i + 1) * d]
    y = (gelu_tanh(x @ w[p + "side.gate"].T) * e) @ w[p + "side.proj"].T
    return norm_plain(y, w[p + "side.norm"], cfg["norm"]["eps"])


# -- the model -----------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """Logits [n, vocab] of a whole sequence from position 0 (and the stream after every layer)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens]
    pos = np.arange(len(tokens))
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "mlstm":
            y = mlstm_mixer(w, p + "mix.", m, x, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(w, p + "mix.", m, x, eps)
        elif layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(w, p + "mix.", m, x, pos, eps)
            y = attention_mixer(w, p + "mix.", m, x, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(w, p + "mlp.", x) if mlp["kind"] == "dense" else moe_ff(w, p + "mlp.", mlp, x)
            x = x + norm_one_plus(y, w[p + "norm2"], eps)
        if cfg.get("token_side"):
            x = x + token_side(w, p, cfg, i, tokens, x)
        streams.append(x.copy())
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
