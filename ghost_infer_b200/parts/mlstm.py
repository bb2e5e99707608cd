"""A matrix memory with exponential gates and a running maximum (the mLSTM of xLSTM).

With h the mixer's input, H heads, keys and queries of K numbers and values of V per head:

    q = Wq h * K^(-1/2),   k = Wk h,   v = Wv h
    i = c tanh((Wi h + bi) / c),   f = log sigmoid(c tanh((Wf h + bf) / c))        one number per head each; c = `gate_cap`
    m_t = max(f_t + m_(t-1), i_t)                                                   m starts at 0
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T               n_t likewise with k_t alone; both start at 0
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's o is divided by its root mean square (eps); the heads side by side are multiplied by a weight of H * V numbers and
by sigmoid(Wg h), and projected: residual += Wo (...).  Per sequence the state is S [H, V, K], n [H, K] and m [H], one float32
row, zero when the sequence starts.  The gates, the maximum, the decays, the recurrence and the norm are 32-bit; the matrix
walks through the kernel that serves the other linear recurrences, with the decays and write strengths made ready beforehand.

Tensor names: prefix + `base` + {q, k, v, i, i.b, f, f.b, g, norm, o} (`base` "mix.").
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .linear_state import _stack
from .registry import register

_KEYS = ("q", "k", "v", "i", "i.b", "f", "f.b", "g", "norm", "o")


@register("mixer", "mlstm")
class MLstm(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.key_dim = int(params["key_dim"])
        self.v_dim = int(params["v_dim"])
        self.cap = float(params["gate_cap"])
        self.eps = float(params["eps"])
        if min(self.heads, self.key_dim, self.v_dim) < 1 or not self.cap > 0:
            raise ValueError("mlstm: sizes and the gates' cap must be positive")
        self.qk_width, self.v_width = self.heads * self.key_dim, self.heads * self.v_dim
        self.s_floats = self.heads * self.key_dim * self.v_dim
        base = str(params.get("base", "mix."))
        self.names = {k: self.tensor_name(k, base + k) for k in _KEYS}

    def weights(self) -> List[WeightSpec]:
        n, d = self.names, self.hidden
        return [WeightSpec(n["q"], (self.qk_width, d)), WeightSpec(n["k"], (self.qk_width, d)), WeightSpec(n["v"], (self.v_width, d)),
                WeightSpec(n["i"], (self.heads, d)), WeightSpec(n["i.b"], (self.heads,)), WeightSpec(n["f"], (self.heads, d)),
                WeightSpec(n["f.b"], (self.heads,)), WeightSpec(n["g"], (self.v_width, d)),
                WeightSpec(n["norm"], (self.v_width,), "ones"), WeightSpec(n["o"], (d, self.v_width))]

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.s_floats + self.heads * (self.key_dim + 1),), torch.float32)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        # one product with 32-bit results: [q | k | v | gate | i | f]
        self.w_in = _stack([rt.place(tensors[n[k]]) for k in ("q", "k", "v", "g", "i", "f")], rt)
        self.w_o = rt.place(tensors[n["o"]])
        f32 = lambda name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()
        self.b_i, self.b_f, self.norm_w = f32(n["i.b"]), f32(n["f.b"]), f32(n["norm"])

    def forward(self, h, residual, step, memory) -> None:
        if memory.state is None:
            raise RuntimeError("the matrix memory was given no per-sequence state")
        qk, vw, H = self.qk_width, self.v_width, self.heads
        with ops.bucket("qkv matmul"):
            proj = linear(h, self.w_in, out_dtype=torch.float32)
        q, k, v = proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vw]
        g0 = 2 * qk + 2 * vw
        with ops.bucket("scan"):
            keep, put, scale = ops.mlstm_gates(q, k, proj[:, g0:g0 + H], proj[:, g0 + H:g0 + 2 * H], self.b_i, self.b_f, self.cap,
                                               self.key_dim ** -0.5, memory.state, self.s_floats, step, H, self.key_dim)
            o = ops.linear_state_gated(q, k, v, memory.state, step, H, self.key_dim, self.v_dim, keep, put)
        with ops.bucket("gated norm"):
            y = ops.scaled_norm_gate(o, scale, proj[:, 2 * qk + vw:g0], self.norm_w, H, self.v_dim, self.eps, self.rt.dtype)
        with ops.bucket("out matmul"):
            linear(y, self.w_o, out=residual, accumulate=True)
