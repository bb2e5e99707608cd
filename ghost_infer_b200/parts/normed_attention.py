"""Grouped-query attention whose queries and keys are normed over their whole projection, then rotated.

With h the mixer's input: q = Wq h (+ bq), k = Wk h (+ bk), v = Wv h (+ bv).  With `qk_norm`, q and k are each divided
by the root mean square of the WHOLE vector (all heads together, before the split into heads) and multiplied by a weight of
that size.  The first `rotary.dims` numbers of every head of q and k turn by the position's angles, pair i by
position * base^(-2i/dims); `rotary.pairing` "adjacent" pairs (2i, 2i+1), "half" pairs (i, i + dims/2); the rest of a head
passes.  score = (q . k) * scale; a query at position i sees keys j <= i, with `window` = w only those with i - j < w;
softmax in 32-bit.  Keys are `head_dim` wide, values `v_head_dim`.  With `out_gate` "sigmoid" the concatenated heads are
multiplied by sigmoid(Wg h) before the output projection.  residual += Wo (heads).

`borrows_kv`: the layer has no key and value tensors; its schedule entry reads another entry's cache (keys as that layer
stored them, after norm and rotation) with its own queries, scale and window.  `cache_window`: what the layer's own cache
keeps when a borrower looks further back than the layer itself (None: every position).

Tensor names: prefix + `base` + {q, q.b, q.norm, k, k.b, k.norm, v, v.b, g, o} (`base` "mix." unless given;
`params["tensor_names"]` replaces any).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import register
from .rope import Rotary

_KEYS = ("q", "q.b", "q.norm", "k", "k.b", "k.norm", "v", "v.b", "g", "o")


@register("mixer", "normed_attention")
class NormedAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.v_dim = int(params.get("v_head_dim") or self.head_dim)
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else None
        self.cache_window = params.get("cache_window", self.window)
        self.bias = bool(params.get("bias", False))
        self.qk_norm = bool(params.get("qk_norm", False))
        self.eps = float(params.get("eps", 1e-6))
        self.out_gate = params.get("out_gate")
        self.borrows_kv = bool(params.get("borrows_kv", False))
        if self.out_gate not in (None, "sigmoid"):
            raise ValueError(f"out_gate must be None or \"sigmoid\", got {self.out_gate!r}")
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv} kv heads")
        if self.cache_window is not None and self.window is not None and int(self.cache_window) < self.window:
            raise ValueError("a cache cannot keep fewer positions than the layer's own window")
        rot = params.get("rotary")
        self.rotary = None
        self.rot_dims = 0
        if rot is not None and int(rot["dims"]) > 0:
            self.rot_dims = int(rot["dims"])
            self.rotary = Rotary({"head_dim": self.head_dim, "rotary_dim": self.rot_dims, "theta": float(rot["base"]),
                                  "pairing": rot.get("pairing", "half")}, prefix)
        self.adjacent = self.rotary is not None and self.rotary.pairing == "adjacent"
        self.q_dim, self.k_dim, self.v_width = self.n_heads * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.v_dim
        base = str(params.get("base", "mix."))
        self.names = {k: self.tensor_name(k, base + k) for k in _KEYS}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        out = [WeightSpec(n["q"], (self.q_dim, self.hidden)), WeightSpec(n["o"], (self.hidden, self.n_heads * self.v_dim))]
        if self.bias:
            out.append(WeightSpec(n["q.b"], (self.q_dim,)))
        if self.qk_norm:
            out.append(WeightSpec(n["q.norm"], (self.q_dim,), "ones"))
        if self.out_gate:
            out.append(WeightSpec(n["g"], (self.q_dim if self.v_dim == self.head_dim else self.n_heads * self.v_dim, self.hidden)))
        if not self.borrows_kv:
            out += [WeightSpec(n["k"], (self.k_dim, self.hidden)), WeightSpec(n["v"], (self.v_width, self.hidden))]
            if self.bias:
                out += [WeightSpec(n["k.b"], (self.k_dim,)), WeightSpec(n["v.b"], (self.v_width,))]
            if self.qk_norm:
                out.append(WeightSpec(n["k.norm"], (self.k_dim,), "ones"))
        return out

    def cache_request(self) -> Optional[CacheRequest]:
        if self.borrows_kv:
            return None
        v = None if self.v_dim == self.head_dim else self.v_dim
        if self.cache_window:
            return CacheRequest("window", self.n_kv, self.head_dim, int(self.cache_window), v)
        return CacheRequest("full", self.n_kv, self.head_dim, None, v)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        return ops.attn_general_decode_plan(n_seqs, max_kv_len, sm_count, self.n_heads, self.n_kv, self.window, None,
                                            self.rt.dtype, self.head_dim, self.v_dim, kv_lens)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        mats = [rt.place(tensors[n["q"]])]
        if not self.borrows_kv:
            mats += [rt.place(tensors[n["k"]]), rt.place(tensors[n["v"]])]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        del mats
        self.w_o = rt.place(tensors[n["o"]])
        self.w_g = rt.place(tensors[n["g"]]) if self.out_gate else None
        # what enters a norm is 32-bit whatever the file stores; biases join the projection's 32-bit sums
        f32 = lambda name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()
        kv = not self.borrows_kv
        self.biases = (f32(n["q.b"]), f32(n["k.b"]) if kv else None, f32(n["v.b"]) if kv else None) if self.bias else (None, None, None)
        self.norms = (f32(n["q.norm"]), f32(n["k.norm"]) if kv else None) if self.qk_norm else (None, None)
        if self.rotary is not None:
            self.rotary.bind(tensors, rt)

    def forward(self, h, residual, step, memory) -> None:
        if memory.k is None:
            raise RuntimeError("attention was given no cache to read")
        if self.borrows_kv == bool(memory.writes):
            raise RuntimeError("a layer that borrows keys and values reads another entry's cache; one that has its own writes it")
        with ops.bucket("qkv matmul"):
            rows = linear(h, self.w_qkv, out_dtype=torch.float32)
        with ops.bucket("rope+cache"):
            table = self.rotary.table(step) if self.rotary is not None else None
            q = ops.qk_prepare(rows, self.rt.dtype, self.biases, self.norms, self.eps, table, self.rot_dims, self.adjacent, step,
                               memory, self.n_heads, 0 if self.borrows_kv else self.n_kv, self.head_dim, self.v_dim)
        with ops.bucket("attention"):
            att = torch.empty((q.shape[0], self.n_heads * self.v_dim), dtype=self.rt.dtype, device=q.device)
            ops.attention_general(q, memory, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim, self.scale, att,
                                  window=self.window, plan=step.plan_of(self))
            if self.out_gate:
                att = ops.gate_mul(att, linear(h, self.w_g, out_dtype=self.rt.dtype), "sigmoid")
        with ops.bucket("out matmul"):
            linear(att, self.w_o, out=residual, accumulate=True)
