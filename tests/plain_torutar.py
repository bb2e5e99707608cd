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


def choice_gaps(h, W, pre, r):
    """Per token, how far the last chosen expert's choice score lies above the first one left out, or, where leaving that
    expert out would hardly matter (its share of the chosen ones' weight is below 3%), infinity; infinity too if all are chosen."""
    z = h @ W[pre + "router"].T
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s = s / s.sum(axis=1, keepdims=True)
    c = s + W[pre + "correction"]
    order = np.argsort(-c, axis=1, kind="stable")
    top = r["top"]
    if top >= c.shape[1]:
        return np.full(h.shape[0], np.inf)
    cs, ss = np.take_along_axis(c, order, axis=1), np.take_along_axis(s, order, axis=1)
    matters = np.maximum(ss[:, top - 1], ss[:, top]) / (ss[:, :top].sum(axis=1) + 1e-20) >= 0.03
    return np.where(matters, cs[:, top - 1] - cs[:, top], np.inf)


def mixture(h, W, pre, mlp, gaps=None):
    ids, w = route(h, W, pre, mlp["router"])
    if gaps is not None:
        gaps.append(choice_gaps(h, W, pre, mlp["router"]))
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


def forward(cfg, W, tokens, return_layers=False, gaps=None):
    """Logits [T, vocab] of one sequence from its first token (float64); optionally the summed streams after every layer.
    `gaps` (a list): receives every routed layer's `choice_gaps`, so that a test can tell where a rounding could flip a choice."""
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
            xs = hyper_sublayer(xs, W, lp, 2, W[lp + "norm2"], eps, lambda h: mixture(h, W, lp + "mlp.", layer["mlp"], gaps))
        after.append(xs.sum(axis=0))
    logits = (rms_unit(xs.sum(axis=0), eps) * W["final.norm"]) @ W["head"].T * cfg["logit_scale"]
    return (logits, np.stack(after)) if return_layers else logits


def bf16_values(a):
    """Rounds to the nearest bfloat16 value (ties to even), kept as float64: a bfloat16 file then holds the weights exactly."""
    f = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return u.view(np.float32).astype(np.float64).reshape(np.shape(a))


def random_weights(cfg, seed=0):
    """Weights for `cfg` (name -> float64 array of bfloat16 values)."""
    rng = np.random.default_rng(seed)
    d, S, out = int(cfg["width"]), int(cfg["streams"]), {}
    taps = int(cfg["canon"]["taps"])

    def put(name, shape, std=None, mean=0.0):
        std = std if std is not None else (1.0 / math.sqrt(shape[-1]) if len(shape) > 1 else 0.5)
        out[name] = bf16_values(rng.standard_normal(shape) * std + mean)

    put("embed", (int(cfg["vocab"]), d), 1.0); put("embed.norm", (d,), 0.1, 1.0)
    put("final.norm", (d,), 0.1, 1.0); put("head", (int(cfg["vocab"]), d))
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        subs = (1, 2) if layer.get("mlp") is not None else (1,)
        for q in subs:
            put(f"{p}norm{q}", (d,), 0.1, 1.0)
            put(f"{p}hc{q}.in", (S,), 0.3, 0.6); put(f"{p}hc{q}.out", (S,), 0.3, 0.8)
            out[f"{p}hc{q}.mix"] = bf16_values(np.eye(S) * 0.9 + rng.standard_normal((S, S)) * 0.15)
            put(f"{p}canon{q}", (d, taps), 0.4); put(f"{p}rg{q}", (d, d)); put(f"{p}rg{q}.b", (d,), 0.5, 0.5)
        x = p + "mix."
        if kind == "attention":
            H, G, n, mv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            put(x + "q", (H * n, d)); put(x + "q.b", (H * n,), 0.3); put(x + "q.norm", (n,), 0.2, 1.3)
            put(x + "sink", (H,), 1.0); put(x + "g", (H, d)); put(x + "o", (d, H * mv)); put(x + "o.b", (d,), 0.2)
            if m.get("kv_from") is None:
                put(x + "k", (G * n, d)); put(x + "k.b", (G * n,), 0.3); put(x + "k.norm", (n,), 0.2, 1.3)
                put(x + "v", (G * mv, d)); put(x + "v.b", (G * mv,), 0.3)
        elif kind == "latent_attention":
            H, n, r, mv, rank, qr = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
            put(x + "dq", (qr, d)); put(x + "dq.norm", (qr,), 0.1, 1.0); put(x + "uq", (H * (n + r), qr))
            put(x + "dkv", (rank + r, d)); put(x + "dkv.norm", (rank,), 0.1, 1.0); put(x + "uk", (H * n, rank))
            put(x + "uv", (H * mv, rank)); put(x + "g", (H * mv, d)); put(x + "o", (d, H * mv))
        else:
            H, n, mv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            put(x + "q", (H * n, d)); put(x + "k", (H * n, d)); put(x + "v", (H * mv, d)); put(x + "g", (H * mv, d))
            put(x + "o", (d, H * mv)); put(x + "norm", (H * mv,), 0.1, 1.0)
            put(x + "i", (H, d), 2.0 / math.sqrt(d)); put(x + "i.b", (H,), 1.0); put(x + "f", (H, d), 2.0 / math.sqrt(d)); put(x + "f.b", (H,), 1.0, 2.0)
        if layer.get("mlp") is not None:
            f, y = layer["mlp"], p + "mlp."
            E = int(f["router"]["experts"])
            put(y + "router", (E, d), 3.0 / math.sqrt(d)); put(y + "correction", (E,), 0.1)
            for e in range(E):
                put(f"{y}e{e}.gate", (int(f["expert"]["ff"]), d), 2.0 / math.sqrt(d)); put(f"{y}e{e}.up", (int(f["expert"]["ff"]), d), 2.0 / math.sqrt(d))
                put(f"{y}e{e}.down", (d, int(f["expert"]["ff"])))
            if f.get("shared") is not None:
                sf = int(f["shared"]["ff"])
                put(y + "shared.gate", (sf, d), 2.0 / math.sqrt(d)); put(y + "shared.up", (sf, d), 2.0 / math.sqrt(d)); put(y + "shared.down", (d, sf))
    return out
