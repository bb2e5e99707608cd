"""Mixers that carry a matrix of state per head from token to token: a gated delta rule and decayed linear attention.

Both walk, per head, S (a key_dim x v_dim matrix of 32-bit numbers, zero when a sequence starts):

    S <- g_t S;   u_t = v_t (or, delta rule: beta_t (v_t - S^T k_t));   S <- S + k_t u_t^T;   o_t = S^T q_t

"gated_delta_rule": q = Wq h and k = Wk h (`qk_heads` heads of key_dim; head a reads query/key head a / (heads / qk_heads)),
v = Wv h (heads of v_dim); each passes a causal convolution over `conv` tokens per channel (no bias; the last tap is the
current token's; zeros before the start) and silu; q and k become unit vectors per head, x / sqrt(sum x^2 + `unit_eps`), q
also times key_dim^(-1/2); beta = sigmoid(Wb h) and g = exp(-exp(A_log) softplus(Wa h + dt_bias)), one per head.  Each
head's o is divided by its root mean square over v_dim (eps), times a weight of v_dim shared by the heads, times
silu(Wg h); residual += Wo (...).  Per sequence: S and the convolution's last `conv` - 1 inputs, one float32 row.

"decayed_linear_attention": q, k = silu(Wq h), silu(Wk h) (heads of key_dim), v = silu(Wv h) (heads of v_dim); g is a
constant per head (`decay`); the concatenated heads are RMS-normed together (weight of heads * v_dim, eps), multiplied by
sigmoid(Wg h), and projected: residual += Wo (...).  Per sequence: S.

The recurrence, decays, gates of the recurrence, unit norms and output norms are 32-bit in both precisions.
Tensor names: prefix + `base` + {q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, norm, g, o} (`base` "mix.").
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import register


def _stack(mats, rt) -> torch.Tensor:
    """Matrices stacked by rows for one product, padded with zero rows to a multiple of 8 rows."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.to(torch.float32) for m in mats]
    w = torch.cat(mats, dim=0)
    pad = (-w.shape[0]) % 8
    if pad:
        w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
    return w.contiguous()


@register("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.qk_heads = int(params["qk_heads"])
        self.key_dim = int(params["key_dim"])
        self.v_dim = int(params["v_dim"])
        self.taps = int(params["conv"])
        self.eps = float(params["eps"])
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        if self.heads % self.qk_heads:
            raise ValueError(f"{self.heads} heads do not divide into {self.qk_heads} query/key heads")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.qk_width, self.v_width = self.qk_heads * self.key_dim, self.heads * self.v_dim
        self.channels = 2 * self.qk_width + self.v_width
        self.s_floats = self.heads * self.key_dim * self.v_dim
        base = str(params.get("base", "mix."))
        keys = ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "a", "A_log", "dt_bias", "norm", "g", "o")
        self.names = {k: self.tensor_name(k, base + k) for k in keys}

    def weights(self) -> List[WeightSpec]:
        n, d = self.names, self.hidden
        return [WeightSpec(n["q"], (self.qk_width, d)), WeightSpec(n["q.conv"], (self.qk_width, self.taps)),
                WeightSpec(n["k"], (self.qk_width, d)), WeightSpec(n["k.conv"], (self.qk_width, self.taps)),
                WeightSpec(n["v"], (self.v_width, d)), WeightSpec(n["v.conv"], (self.v_width, self.taps)),
                WeightSpec(n["b"], (self.heads, d)), WeightSpec(n["A_log"], (self.heads,)),
                WeightSpec(n["norm"], (self.v_dim,), "ones"), WeightSpec(n["a"], (self.heads, d)),
                WeightSpec(n["dt_bias"], (self.heads,)), WeightSpec(n["g"], (self.v_width, d)),
                WeightSpec(n["o"], (d, self.v_width))]

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.s_floats + (self.taps - 1) * self.channels,), torch.float32)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        # one product: [q | k | v | gate | beta | decay]; the convolved channels come first
        self.w_in = _stack([rt.place(tensors[n[k]]) for k in ("q", "k", "v", "g", "b", "a")], rt)
        self.w_o = rt.place(tensors[n["o"]])
        cw = [rt.place(tensors[n[k]]) for k in ("q.conv", "k.conv", "v.conv")]
        if len({c.dtype for c in cw}) > 1:
            cw = [c.to(torch.float32) for c in cw]
        self.conv_w = torch.cat(cw, dim=0).contiguous()
        self.conv_b = torch.zeros((self.channels,), dtype=self.conv_w.dtype, device=rt.device)     # the design has no bias
        # the recurrence's constants and the norm's weight enter 32-bit arithmetic: kept as 32-bit values
        f32 = lambda name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()
        self.a_log, self.dt_bias, self.norm_w = f32(n["A_log"]), f32(n["dt_bias"]), f32(n["norm"])

    def forward(self, h, residual, step, memory) -> None:
        if memory.state is None:
            raise RuntimeError("the delta rule was given no per-sequence state")
        C, qk, vw, H = self.channels, self.qk_width, self.v_width, self.heads
        with ops.bucket("qkv matmul"):
            proj = linear(h, self.w_in, out_dtype=self.rt.dtype)
        with ops.bucket("conv"):
            conv = ops.mamba2_conv(proj, self.conv_w, self.conv_b, memory.state, step, 0, C, self.taps, self.s_floats)
        with ops.bucket("scan"):
            o = ops.linear_state(conv[:, :qk], conv[:, qk:2 * qk], conv[:, 2 * qk:], memory.state, step, H, self.qk_heads,
                                 self.key_dim, self.v_dim, self.a_log, decay_in=proj[:, C + vw + H:C + vw + 2 * H],
                                 dt_bias=self.dt_bias, beta_in=proj[:, C + vw:C + vw + H], unit_norm=True,
                                 norm_eps=self.unit_eps, q_scale=self.key_dim ** -0.5, delta=True)
        with ops.bucket("gated norm"):
            y = ops.norm_gate(o, proj[:, C:C + vw], self.norm_w, self.v_dim, self.eps, "silu", self.rt.dtype)
        with ops.bucket("out matmul"):
            linear(y, self.w_o, out=residual, accumulate=True)


@register("mixer", "decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.key_dim = int(params["key_dim"])
        self.v_dim = int(params["v_dim"])
        self.eps = float(params["eps"])
        self.decay = tuple(float(g) for g in params["decay"])
        if len(self.decay) != self.heads:
            raise ValueError(f"{len(self.decay)} decays for {self.heads} heads")
        self.qk_width, self.v_width = self.heads * self.key_dim, self.heads * self.v_dim
        base = str(params.get("base", "mix."))
        self.names = {k: self.tensor_name(k, base + k) for k in ("q", "k", "v", "g", "o", "norm")}

    def weights(self) -> List[WeightSpec]:
        n, d = self.names, self.hidden
        return [WeightSpec(n["q"], (self.qk_width, d)), WeightSpec(n["k"], (self.qk_width, d)), WeightSpec(n["v"], (self.v_width, d)),
                WeightSpec(n["g"], (self.v_width, d)), WeightSpec(n["o"], (d, self.v_width)),
                WeightSpec(n["norm"], (self.v_width,), "ones")]

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.heads * self.key_dim * self.v_dim,), torch.float32)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        self.w_in = _stack([rt.place(tensors[n[k]]) for k in ("q", "k", "v", "g")], rt)
        self.w_o = rt.place(tensors[n["o"]])
        self.norm_w = tensors[n["norm"]].to(device=rt.device, dtype=torch.float32).contiguous()
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(device=rt.device, dtype=torch.float32)

    def forward(self, h, residual, step, memory) -> None:
        if memory.state is None:
            raise RuntimeError("linear attention was given no per-sequence state")
        qk, vw = self.qk_width, self.v_width
        with ops.bucket("qkv matmul"):
            proj = linear(h, self.w_in, out_dtype=self.rt.dtype)
        with ops.bucket("scan"):
            o = ops.linear_state(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vw], memory.state, step, self.heads,
                                 self.heads, self.key_dim, self.v_dim, self.decay_dev, in_act=True)
        with ops.bucket("gated norm"):
            y = ops.norm_gate(o, proj[:, 2 * qk + vw:2 * qk + 2 * vw], self.norm_w, vw, self.eps, "sigmoid", self.rt.dtype)
        with ops.bucket("out matmul"):
            linear(y, self.w_o, out=residual, accumulate=True)
