"""A plain, slow implementation of the Nuzinex decoder, used as the oracle of its tests.

Whole sequences, no cache, no batch, one function per mechanism, numpy only, float64 by default.  It shares no code
with the package under test.  Notation: T tokens, d the model's width; a matrix W is stored [out, in] and applied to
row vectors as h @ W.T; `w` is a dict of a part's tensors by their short names.

The design.  x = E[token].  A layer reads the stream itself and norms what its sublayers give back:
x += s1 * rms(mixer(x)), then (if the layer has a feed-forward) x += s2 * rms(ff(x)), s1 and s2 learned vectors; after
that every layer adds a per-token input of its own: a slice of a second embedding table, gated by a small projection
of x, projected back to d and divided by its root mean square.  The mixer is one of: attention inside a sliding window
(biases, a norm over the whole query and key projections, rotation of neighbouring pairs; a layer may borrow another
layer's keys and values); two mixers side by side whose outputs are added with constant weights (causal attention with
a sigmoid gate on its heads' outputs, and a gated delta rule with short convolutions); or linear attention with a
constant decay per head.  The feed-forward is W_down gelu(W_up h).  A final norm and an output matrix.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------------------------
# files
def read_safetensors(path, dtype=np.float64):
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(dtype)
        elif info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(dtype)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = arr.reshape(info["shape"])
    return out


def read_model(model_dir, dtype=np.float64):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors", dtype)


# ---------------------------------------------------------------------------------------------------------------
# small functions
def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(np.asarray(z, dtype=np.float64) / math.sqrt(2.0)))


# ---------------------------------------------------------------------------------------------------------------
# rotation
def rotate(x, positions, rot, layout):
    """x [T, heads, dim]; the first `rot["dims"]` numbers of each head turn by angle p * base^(-2i/dims) in pair i.
    layout "neighbours": pair i is (2i, 2i+1); "halves": pair i is (i, i + dims/2)."""
    n = int(rot["dims"])
    half = n // 2
    freq = float(rot["base"]) ** (-2.0 * np.arange(half) / n)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if layout == "neighbours":
        a, b = x[..., 0:n:2], x[..., 1:n:2]
        out[..., 0:n:2] = a * c - b * s
        out[..., 1:n:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:n]
        out[..., :half] = a * c - b * s
        out[..., half:n] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------------------------
# softmax attention
def keys_and_values(h, w, m, eps, layout, biased):
    """The cache's view of a layer: keys after norm and rotation [T, G, dim], values [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w["k"].T
    v = h @ w["v"].T
    if biased:
        k, v = k + w["k.b"], v + w["v.b"]
    k = rms_norm(k, w["k.norm"], eps)                  # one norm over all heads' rows together
    k = rotate(k.reshape(T, G, dim), np.arange(T), m["rot"], layout)
    return k, v.reshape(T, G, vdim)


def softmax_heads(h, w, m, eps, layout, biased, kv=None):
    """Concatenated heads [T, H * vdim] of softmax attention.  `m["mask"]["size"]` = s: query i sees keys j with
    0 <= i - j < s; without it every j <= i.  `kv`: keys and values borrowed from another layer."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w["q"].T
    if biased:
        q = q + w["q.b"]
    q = rms_norm(q, w["q.norm"], eps)
    q = rotate(q.reshape(T, H, dim), np.arange(T), m["rot"], layout)
    k, v = kv if kv is not None else keys_and_values(h, w, m, eps, layout, biased)
    size = m["mask"]["size"] if m.get("mask") else None
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) if size is None else ((j <= i) & (i - j < size))
    out = np.zeros((T, H, vdim), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        out[:, a] = p @ v[:, g]
    return out.reshape(T, H * vdim)


def window_attention(h, w, m, eps, kv=None):
    return softmax_heads(h, w, m, eps, "neighbours", True, kv) @ w["o"].T


def gated_attention(h, w, m, eps):
    heads = softmax_heads(h, w, m, eps, "halves", False)
    return (heads * sigmoid(h @ w["g"].T)) @ w["o"].T


# ---------------------------------------------------------------------------------------------------------------
# recurrent mixers
def short_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: out[t, c] = sum_j taps_w[c, j] u[t - (taps - 1) + j, c], zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=u.dtype), u], axis=0)
    out = np.zeros_like(u)
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j][None, :]
    return out


def delta_rule(h, w, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, dim)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, dim)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)                                                      # [T, H]
    decay = np.exp(-np.exp(w["A_log"])[None, :] * softplus(h @ w["a"].T + w["dt_bias"][None, :]))
    o = np.zeros((T, H, vdim), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((dim, vdim), dtype=h.dtype)
        for t in range(T):
            S = decay[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, a] = S.T @ q[t, g]
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * w["norm"]
    gate = silu(h @ w["g"].T).reshape(T, H, vdim)
    return (o * gate).reshape(T, H * vdim) @ w["o"].T


def side_by_side(h, w, m, eps):
    left = gated_attention(h, under(w, "left."), m["left"], eps)
    right = delta_rule(h, under(w, "right."), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def lightning(h, w, m, eps):
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, dim)
    k = silu(h @ w["k"].T).reshape(T, H, dim)
    v = silu(h @ w["v"].T).reshape(T, H, vdim)
    o = np.zeros((T, H, vdim), dtype=h.dtype)
    for a in range(H):
        S = np.zeros((dim, vdim), dtype=h.dtype)
        for t in range(T):
            S = m["decay"][a] * S + np.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = rms_norm(o.reshape(T, H * vdim), w["norm"], eps)
    return (o * sigmoid(h @ w["g"].T)) @ w["o"].T


# ---------------------------------------------------------------------------------------------------------------
# the rest of a layer
def dense_ff(h, w):
    return gelu_erf(h @ w["up"].T) @ w["down"].T


def token_side(x, tokens, table, w, layer, dim, eps):
    e = table[np.asarray(tokens)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps) * w["norm"]


def under(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  `layers_out`: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = weights["embed"][tokens]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        w = under(weights, f"l{i}.")
        m = layer["mixer"]
        wm = under(w, "mix.")
        if layer["type"] == "attention":
            if m.get("kv_from") is not None:
                y = window_attention(x, wm, m, eps, kv=kept[m["kv_from"]])
            else:
                kept[i] = keys_and_values(x, wm, m, eps, "neighbours", True)
                y = window_attention(x, wm, m, eps)
        elif layer["type"] == "parallel":
            y = side_by_side(x, wm, m, eps)
        elif layer["type"] == "lightning":
            y = lightning(x, wm, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w["norm1"], eps) * w["ls1"]
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(x, under(w, "mlp.")), w["norm2"], eps) * w["ls2"]
        x = x + token_side(x, tokens, weights["side.embed"], under(w, "side."), i, cfg["token_side"]["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T


# ---------------------------------------------------------------------------------------------------------------
# random models
def bf16_values(a, dtype=np.float64):
    """`a` rounded (to nearest, ties to even) to values a bfloat16 holds."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32)
    return r.view(np.float32).astype(dtype).reshape(a.shape)


def random_weights(cfg, seed=0, dtype=np.float64):
    """Weights for `cfg`, rounded to bfloat16 values so that a bfloat16 file holds them exactly."""
    rng = np.random.default_rng(seed)
    d, out = int(cfg["width"]), {}

    def put(name, shape, std=None, mean=0.0):
        std = std if std is not None else 1.0 / math.sqrt(shape[-1]) if len(shape) > 1 else 0.5
        out[name] = bf16_values(rng.standard_normal(shape) * std + mean, dtype)

    def softmax_tensors(p, m, biased, gated, own_kv=True):
        H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        put(p + "q", (H * dk, d)); put(p + "q.norm", (H * dk,), 0.2, 1.3); put(p + "o", (d, H * dv))
        if biased:
            put(p + "q.b", (H * dk,), 0.3)
        if gated:
            put(p + "g", (H * dv, d))
        if own_kv:
            put(p + "k", (G * dk, d)); put(p + "v", (G * dv, d)); put(p + "k.norm", (G * dk,), 0.2, 1.3)
            if biased:
                put(p + "k.b", (G * dk,), 0.3); put(p + "v.b", (G * dv,), 0.3)

    put("embed", (int(cfg["vocab"]), d), 1.0)
    put("side.embed", (int(cfg["vocab"]), int(cfg["token_side"]["dim"]) * len(cfg["layers"])), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        put(p + "norm1", (d,), 0.1, 1.0); put(p + "ls1", (d,), 0.1, 0.5)
        if layer["type"] == "attention":
            softmax_tensors(p + "mix.", m, True, False, m.get("kv_from") is None)
        elif layer["type"] == "parallel":
            softmax_tensors(p + "mix.left.", m["left"], False, True)
            r, q = m["right"], p + "mix.right."
            H, G, dk, dv, taps = int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r["conv"])
            put(q + "q", (G * dk, d)); put(q + "q.conv", (G * dk, taps), 0.6); put(q + "k", (G * dk, d)); put(q + "k.conv", (G * dk, taps), 0.6)
            put(q + "v", (H * dv, d)); put(q + "v.conv", (H * dv, taps), 0.6); put(q + "b", (H, d)); put(q + "a", (H, d))
            put(q + "A_log", (H,), 0.5, -0.5); put(q + "dt_bias", (H,), 0.5, -1.0); put(q + "norm", (dv,), 0.1, 1.0)
            put(q + "g", (H * dv, d)); put(q + "o", (d, H * dv))
        else:
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            put(p + "mix.q", (H * dk, d)); put(p + "mix.k", (H * dk, d)); put(p + "mix.v", (H * dv, d)); put(p + "mix.g", (H * dv, d))
            put(p + "mix.o", (d, H * dv)); put(p + "mix.norm", (H * dv,), 0.1, 1.0)
        if layer.get("mlp"):
            f = int(layer["mlp"]["ff"])
            put(p + "norm2", (d,), 0.1, 1.0); put(p + "ls2", (d,), 0.1, 0.5)
            put(p + "mlp.up", (f, d)); put(p + "mlp.down", (d, f))
        sd = int(cfg["token_side"]["dim"])
        put(p + "side.gate", (sd, d)); put(p + "side.proj", (d, sd)); put(p + "side.norm", (d,), 0.05, 0.3)
    put("final.norm", (d,), 0.1, 1.0)
    put("head", (int(cfg["vocab"]), d))
    return out


def write_safetensors_bf16(path, tensors):
    """Writes float arrays as bfloat16 (the values must be bfloat16 values already) in the safetensors layout."""
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        raw = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
