"""A plain, slow Torutar decoder in numpy float64: one function per mechanism, whole sequences at once.

It shares no code with the library: the tests compare the library's logits and intermediate results with what these
functions give for the same configuration dict and the same tensors (name -> array).  Notation: T tokens, d the width,
H heads; matrices are stored [out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def causal_conv_added(h, w):
    """h + conv(h): conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start.  h [T, d], w [d, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = h.copy()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += h[:T - back] * w[:, j]
    return out


def rotate(x, positions, dims, base, layout):
    """Turns the first `dims` numbers of the last axis of x [T, ..., n] by the positions' angles."""
    if dims == 0:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]            # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = x.copy()
    if layout == "half":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half], out[..., half:dims] = a * c - b * s, b * c + a * s
    else:                                                                            # neighbours (2i, 2i + 1)
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    return out


def visible(T, size=None, keep_first=0):
    """[T, T] booleans: query i sees key j."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok &= (i - j < size) | (j < keep_first)
    return ok


def softmax_attention(q, k, v, scale, mask, sink=None):
    """q [T, H, n], k [T, G, n], v [T, G, m] -> [T, H, m]; `sink` [H]: one more term of the denominator per head."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(mask, s, -np.inf)
        top = s.max(axis=1, keepdims=True)
        if sink is not None:
            top = np.maximum(top, sink[h])
        p = np.exp(s - top)
        den = p.sum(axis=1, keepdims=True)
        if sink is not None:
            den = den + np.exp(sink[h] - top)
        out[:, h] = (p / den) @ v[:, g]
    return out


def windowed_attention_kv(h, positions, W, pre, m, eps):
    """Keys (normed, rotated) and values (divided by their root mean square) of a layer that has its own."""
    T, G, n, mv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).reshape(T, G, n)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).reshape(T, G, mv)
    k = rms_unit(k, eps) * W[pre + "k.norm"]
    k = rotate(k, positions, m["rot"]["dims"], m["rot"]["base"], "half")
    return k, rms_unit(v, eps)


def windowed_attention(h, positions, W, pre, m, eps, kv):
    T, H, n = h.shape[0], m["heads"], m["dim"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).reshape(T, H, n)
    q = rms_unit(q, eps) * W[pre + "q.norm"]
    q = rotate(q, positions, m["rot"]["dims"], m["rot"]["base"], "half")
    k, v = kv
    mask = visible(T, m["mask"]["size"], m["mask"]["keep_first"])
    o = softmax_attention(q, k, v, m["scale"], mask, W[pre + "sink"])
    o = o * sigmoid(h @ W[pre + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ W[pre + "o"].T + W[pre + "o.b"]


def latent_attention(h, positions, W, pre, m, eps):
    T, H, n, r, mv, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_unit(h @ W[pre + "dq"].T, eps) * W[pre + "dq.norm"]
    q = (cq @ W[pre + "uq"].T).reshape(T, H, n + r)
    down = h @ W[pre + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * W[pre + "dkv.norm"]
    k_rot = rotate(down[:, rank:], positions, m["rot"]["dims"], m["rot"]["base"], "adjacent")        # [T, r], all heads share it
    q_rot = rotate(q[:, :, n:], positions, m["rot"]["dims"], m["rot"]["base"], "adjacent")
    k_plain = (c @ W[pre + "uk"].T).reshape(T, H, n)
    v = (c @ W[pre + "uv"].T).reshape(T, H, mv)
    qq = np.concatenate([q[:, :, :n], q_rot], axis=2)
    kk = np.concatenate([k_plain, np.broadcast_to(k_rot[:, None, :], (T, H, r))], axis=2)
    o = softmax_attention(qq, kk, v, m["scale"], visible(T))
    o = o.reshape(T, -1) * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def mlstm(h, W, pre, m, eps, state=None):
    """The matrix memory with a running maximum.  `state` (S [H, n, mv], n [H, n], m [H]) is carried in and returned."""
    T, H, n, mv, cap = h.shape[0], m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[pre + "q"].T).reshape(T, H, n) * n ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, n)
    v = (h @ W[pre + "v"].T).reshape(T, H, mv)
    gi = cap * np.tanh((h @ W[pre + "i"].T + W[pre + "i.b"]) / cap)                  # [T, H] log input gate
    gf = log_sigmoid(cap * np.tanh((h @ W[pre + "f"].T + W[pre + "f.b"]) / cap))     # [T, H] log forget gate
    if state is None:
        state = (np.zeros((H, n, mv)), np.zeros((H, n)), np.zeros(H))
    S, nn, mm = (a.copy() for a in state)
    o = np.zeros((T, H, mv))
    for t in range(T):
        for a in range(H):
            m_new = max(gf[t, a] + mm[a], gi[t, a])
            keep, put = math.exp(gf[t, a] + mm[a] - m_new), math.exp(gi[t, a] - m_new)
            S[a] = keep * S[a] + put * np.outer(k[t, a], v[t, a])
            nn[a] = keep * nn[a] + put * k[t, a]
            mm[a] = m_new
            o[t, a] = (S[a].T @ q[t, a]) / (max(abs(nn[a] @ q[t, a]), math.exp(-m_new)) + 1e-6)
    o = rms_unit(o, eps).reshape(T, H * mv) * W[pre + "norm"] * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T, (S, nn, mm)


def clamped_expert(h, W, pre, limit):
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def route(h, W, pre, r):
    """Chosen experts [T, top] and their weights [T, top]."""
    z = h @ W[pre + "router"].T
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s = s / s.sum(axis=1, keepdims=True)
    choice = s + W[pre + "correction"]
    ids = np.argsort(-choice, axis=1, kind="stable")[:, :r["top"]]
    w = np.take_along_axis(s, ids, axis=1)
    w = w / (w.sum(axis=1, keepdims=True) + 1e-20) * r["scale"]
    return ids, w


def mixture(h, W, pre, mlp):
    ids, w = route(h, W, pre, mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t], w[t]):
            out[t] += we * clamped_expert(h[t:t + 1], W, f"{pre}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out += clamped_expert(h, W, pre + "shared.", mlp["shared"]["limit"])
    return out


def hyper_sublayer(xs, W, lp, q, norm_w, eps, run):
    """One sublayer across the streams xs [s, T, d]: read, norm, gate, input convolution, sublayer, write back."""
    u = np.tensordot(W[f"{lp}hc{q}.in"], xs, axes=(0, 0))
    h = rms_unit(u, eps) * norm_w
    gate = sigmoid(h @ W[f"{lp}rg{q}"].T + W[f"{lp}rg{q}.b"])
    y = run(causal_conv_added(h, W[f"{lp}canon{q}"])) * gate
    mixed = np.tensordot(W[f"{lp}hc{q}.mix"].T, xs, axes=(1, 0))                      # new stream t = sum_s mix[s, t] x_s
    return mixed + W[f"{lp}hc{q}.out"][:, None, None] * y[None]


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token (float64); optionally the summed streams after every layer."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = np.arange(T)
    x = rms_unit(W["embed"][np.asarray(tokens)], eps) * W["embed.norm"]
    xs = np.stack([x] * cfg["streams"])
    kept = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        lp, m = f"l{i}.", layer["mixer"]
        pre = lp + "mix."

        def mixer(h):
            if layer["type"] == "mlstm":
                return mlstm(h, W, pre, m, eps)[0]
            if layer["type"] == "latent_attention":
                return latent_attention(h, positions, W, pre, m, eps)
            if m.get("kv_from") is None:
                kept[i] = windowed_attention_kv(h, positions, W, pre, m, eps)
            return windowed_attention(h, positions, W, pre, m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])

        xs = hyper_sublayer(xs, W, lp, 1, W[lp + "norm1"], eps, mixer)
        if layer.get("mlp") is not None:
            xs = hyper_sublayer(xs, W, lp, 2, W[lp + "norm2"], eps, lambda h: mixture(h, W, lp + "mlp.", layer["mlp"]))
        after.append(xs.sum(axis=0))
    logits = (rms_unit(xs.sum(axis=0), eps) * W["final.norm"]) @ W["head"].T * cfg["logit_scale"]
    return (logits, np.stack(after)) if return_layers else logits
