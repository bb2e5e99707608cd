"""Grouped-query attention normed head by head, inside a window that may keep the first positions, with a sink and gated heads.

With h the mixer's input, H query heads, G key/value heads (head a reads key/value head a / (H / G)), keys of `head_dim` and
values of `v_head_dim` numbers:

    q = Wq h (+ bq),  k = Wk h (+ bk),  v = Wv h (+ bv)
    `qk_norm`: every head of q and of k is divided by its own root mean square and multiplied by a weight of head_dim numbers
               that all heads share (before the rotation);  `v_norm`: every head of v is divided by its root mean square, and
               cached so
    the first `rotary.dims` numbers of every head of q and k turn by position * base^(-2i / dims), pairs (i, i + dims / 2)
               (`rotary.pairing` "half") or (2i, 2i + 1) ("adjacent"); the rest of a head passes
    score = (q . k) * scale;  position i sees j <= i with i - j < `window` or j < `keep_first` (kept positions keep their
               true positions); softmax in 32-bit, with `sink` a learned number per head whose exponential joins the
               denominator without key or value
    `head_gate`: head a's output is multiplied by sigmoid(Wg h)_a, one number per head
    residual += Wo (heads) (+ bo)

`borrows_kv`: the layer has no key and value tensors; its schedule entry reads another entry's cache with its own queries,
window and everything else.  `cache_window` / `cache_keep_first`: what the layer's own cache keeps when a borrower looks
further back than the layer itself.

Tensor names: prefix + `base` + {q, q.b, q.norm, k, k.b, k.norm, v, v.b, sink, g, o, o.b} (`base` "mix.").
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .linear_state import _stack
from .registry import register
from .rope import Rotary

_KEYS = ("q", "q.b", "q.norm", "k", "k.b", "k.norm", "v", "v.b", "sink", "g", "o", "o.b")


@register("mixer", "head_normed_attention")
class HeadNormedAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.v_dim = int(params.get("v_head_dim") or self.head_dim)
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else None
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.cache_window = params.get("cache_window", self.window)
        self.cache_keep_first = int(params.get("cache_keep_first", self.keep_first) or 0)
        self.bias = bool(params.get("bias", False))
        self.qk_norm = bool(params.get("qk_norm", False))
        self.v_norm = bool(params.get("v_norm", False))
        self.has_sink = bool(params.get("sink", False))
        self.head_gate = bool(params.get("head_gate", False))
        self.eps = float(params.get("eps", 1e-6))
        self.borrows_kv = bool(params.get("borrows_kv", False))
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv} kv heads")
        if self.cache_window is not None and (self.window is None or int(self.cache_window) < self.window):
            raise ValueError("a cache cannot keep fewer positions than the layer's own window")
        if self.cache_window is not None and self.cache_keep_first < self.keep_first:
            raise ValueError("a cache cannot keep fewer first positions than the layer itself sees")
        rot = params.get("rotary")
        self.rotary, self.rot_dims = None, 0
        if rot is not None and int(rot["dims"]) > 0:
            self.rot_dims = int(rot["dims"])
            self.rotary = Rotary({"head_dim": self.head_dim, "rotary_dim": self.rot_dims, "theta": float(rot["base"]),
                                  "pairing": rot.get("pairing", "half")}, prefix)
        self.adjacent = self.rotary is not None and self.rotary.pairing == "adjacent"
        self.q_dim, self.k_dim, self.v_width = self.n_heads * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.v_dim
        base = str(params.get("base", "mix."))
        self.names = {k: self.tensor_name(k, base + k) for k in _KEYS}

    def weights(self) -> List[WeightSpec]:
        n, kv = self.names, not self.borrows_kv
        out = [WeightSpec(n["q"], (self.q_dim, self.hidden)), WeightSpec(n["o"], (self.hidden, self.n_heads * self.v_dim))]
        if kv:
            out += [WeightSpec(n["k"], (self.k_dim, self.hidden)), WeightSpec(n["v"], (self.v_width, self.hidden))]
        if self.bias:
            out += [WeightSpec(n["q.b"], (self.q_dim,)), WeightSpec(n["o.b"], (self.hidden,))]
            if kv:
                out += [WeightSpec(n["k.b"], (self.k_dim,)), WeightSpec(n["v.b"], (self.v_width,))]
        if self.qk_norm:
            out.append(WeightSpec(n["q.norm"], (self.head_dim,), "ones"))
            if kv:
                out.append(WeightSpec(n["k.norm"], (self.head_dim,), "ones"))
        if self.has_sink:
            out.append(WeightSpec(n["sink"], (self.n_heads,)))
        if self.head_gate:
            out.append(WeightSpec(n["g"], (self.n_heads, self.hidden)))
        return out

    def cache_request(self) -> Optional[CacheRequest]:
        if self.borrows_kv:
            return None
        v = None if self.v_dim == self.head_dim else self.v_dim
        if self.cache_window:
            return CacheRequest("window", self.n_kv, self.head_dim, int(self.cache_window), v, keep_first=self.cache_keep_first)
        return CacheRequest("full", self.n_kv, self.head_dim, None, v)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        return ops.attn_general_decode_plan(n_seqs, max_kv_len, sm_count, self.n_heads, self.n_kv, self.window, None,
                                            self.rt.dtype, self.head_dim, self.v_dim, kv_lens, keep_first=self.keep_first)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n, kv = self.names, not self.borrows_kv
        mats = [rt.place(tensors[n["q"]])]
        if kv:
            mats += [rt.place(tensors[n["k"]]), rt.place(tensors[n["v"]])]
        if self.head_gate:
            mats.append(rt.place(tensors[n["g"]]))
        self.w_in = _stack(mats, rt)          # one product with 32-bit results: [q | k | v | one gate per head]
        del mats
        self.w_o = rt.place(tensors[n["o"]])
        # what enters a norm or the softmax is 32-bit whatever the file stores; biases join the projection's 32-bit sums
        f32 = lambda name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()
        self.biases = (f32(n["q.b"]), f32(n["k.b"]) if kv else None, f32(n["v.b"]) if kv else None) if self.bias else (None, None, None)
        self.b_o = f32(n["o.b"]) if self.bias else None
        self.norm_w = (f32(n["q.norm"]), f32(n["k.norm"]) if kv else None) if self.qk_norm else (None, None)
        self.sinks = f32(n["sink"]) if self.has_sink else None
        if self.rotary is not None:
            self.rotary.bind(tensors, rt)

    def forward(self, h, residual, step, memory) -> None:
        if memory.k is None:
            raise RuntimeError("attention was given no cache to read")
        if self.borrows_kv == bool(memory.writes):
            raise RuntimeError("a layer that borrows keys and values reads another entry's cache; one that has its own writes it")
        n_kv = 0 if self.borrows_kv else self.n_kv
        with ops.bucket("qkv matmul"):
            rows = linear(h, self.w_in, out_dtype=torch.float32)
        with ops.bucket("rope+cache"):
            table = self.rotary.table(step) if self.rotary is not None else None
            q = ops.head_prepare(rows, self.rt.dtype, self.biases, self.norm_w, (self.qk_norm, self.qk_norm, self.v_norm), self.eps, table,
                                 self.rot_dims, self.adjacent, step, memory, self.n_heads, n_kv, self.head_dim, self.v_dim)
        with ops.bucket("attention"):
            att = torch.empty((q.shape[0], self.n_heads * self.v_dim), dtype=self.rt.dtype, device=q.device)
            ops.attention_general(q, memory, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim, self.scale, att,
                                  window=self.window, sinks=self.sinks, plan=step.plan_of(self), keep_first=self.keep_first)
            if self.head_gate:
                g0 = self.q_dim + (0 if self.borrows_kv else self.k_dim + self.v_width)
                att = ops.head_gate(att, rows[:, g0:g0 + self.n_heads], self.n_heads, self.v_dim)
        with ops.bucket("out matmul"):
            if self.b_o is not None:
                ops.settle(residual)
                ops.add_row_bias(residual, self.b_o)
            linear(att, self.w_o, out=residual, accumulate=True)
