"""Causal attention whose keys and values come out of one low-rank latent per token ("latent attention").

With h the mixer's input, H heads, a head's query and key made of `dim` unrotated and `rot_dim` rotated numbers, values
of `v_dim` numbers, a latent of `rank` numbers and a query latent of `q_rank`:

    cq = rmsnorm(W_dq h) * w_dq_norm                      q = W_uq cq, per head [dim | rot_dim]
    [a | kr] = W_dkv h   (rank | rot_dim numbers)         c = rmsnorm(a) * w_dkv_norm
    k_h = W_uk,h c       v_h = W_uv,h c                   kr: one rotated key part shared by all heads
    score_h(i, j) = (q_h,unrot(i) . k_h(j) + rot(q_h,rot(i)) . rot(kr(j))) * scale,   j <= i,   softmax,   out = W_o [sum p v_h]

The position encoding (`params["position"]`, a rotary part) turns the rotated parts only; values are not rotated; `scale`
is used as given.  With `out_gate` "sigmoid" the heads side by side are multiplied by sigmoid(W_g h) (tensor "g") before W_o.
Only c and the rotated kr are cached: one row [c | kr] per position, shared by all heads and serving
as key and as value (`CacheRequest(values_in_keys=True)`).  To attend over such rows a head's unrotated query is carried
onto the latent, qa_h = W_uk,h^T q_h,unrot (so that qa_h . c = q_h,unrot . k_h), the attention runs with every head
reading the same rows, its result per head is a weighted sum of latents, and W_uv,h turns that into the head's values.
Norms, angles, scores and softmax are 32-bit.

Tensor names: prefix + "mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}" unless `params["tensor_names"]` gives others for the keys
"dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o".
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import lookup, register

_DEFAULT_NAMES = {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm",
                  "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o", "g": "mix.g"}


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.dim = int(params["head_dim"])              # unrotated numbers of a head's query and key
        self.rot_dim = int(params["rot_dim"])           # rotated numbers (the shared key part's width)
        self.v_dim = int(params["v_head_dim"])
        self.rank = int(params["kv_rank"])
        self.q_rank = int(params["q_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.out_gate = params.get("out_gate")
        if self.out_gate not in (None, "sigmoid"):
            raise ValueError(f"out_gate must be None or \"sigmoid\", got {self.out_gate!r}")
        if min(self.n_heads, self.dim, self.v_dim, self.rank, self.q_rank) < 1 or self.rot_dim < 0:
            raise ValueError("latent attention: sizes must be positive")
        pos = params.get("position")
        self.position = lookup("position", pos.kind)(pos.params, prefix) if pos is not None and self.rot_dim > 0 else None
        self.rot = int(self.position.rotary_dim) if self.position is not None else 0     # how many of rot_dim turn
        if self.rot > self.rot_dim:
            raise ValueError(f"latent attention: {self.rot} numbers cannot turn in a rotated part of {self.rot_dim}")
        if self.position is not None and getattr(self.position, "pairing", "adjacent") != "adjacent":
            raise ValueError("latent attention turns neighbouring pairs: the position encoding must pair (2i, 2i + 1)")
        self.names = {k: self.tensor_name(k, v) for k, v in _DEFAULT_NAMES.items()}

    def weights(self) -> List[WeightSpec]:
        n, H = self.names, self.n_heads
        gate = [WeightSpec(n["g"], (H * self.v_dim, self.hidden))] if self.out_gate else []
        return gate + [WeightSpec(n["dq"], (self.q_rank, self.hidden)), WeightSpec(n["dq_norm"], (self.q_rank,), "ones"),
                WeightSpec(n["uq"], (H * (self.dim + self.rot_dim), self.q_rank)),
                WeightSpec(n["dkv"], (self.rank + self.rot_dim, self.hidden)), WeightSpec(n["dkv_norm"], (self.rank,), "ones"),
                WeightSpec(n["uk"], (H * self.dim, self.rank)), WeightSpec(n["uv"], (H * self.v_dim, self.rank)),
                WeightSpec(n["o"], (self.hidden, H * self.v_dim))]

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest("full", 1, self.rank + self.rot_dim, None, self.rank, values_in_keys=True)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        return ops.attn_latent_decode_plan(n_seqs, max_kv_len, sm_count, self.n_heads, self.rank, self.rot_dim, self.rt.dtype)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n, H = self.names, self.n_heads
        dq, dkv = rt.place(tensors[n["dq"]]), rt.place(tensors[n["dkv"]])
        if dq.dtype != dkv.dtype:
            dq, dkv = dq.to(torch.float32), dkv.to(torch.float32)
        self.w_down = torch.cat([dq, dkv], dim=0).contiguous()       # one product: [query latent | latent | rotary key part]
        del dq, dkv
        self.w_uq = rt.place(tensors[n["uq"]])
        self.w_o = rt.place(tensors[n["o"]])
        self.w_g = rt.place(tensors[n["g"]]) if self.out_gate else None
        # per head: W_uk,h^T as [rank, dim] (rows of the carried query), W_uv,h as [v_dim, rank]
        self.w_uk_t = rt.place(tensors[n["uk"]]).view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = rt.place(tensors[n["uv"]]).view(H, self.v_dim, self.rank).contiguous()
        qn, cn = rt.place(tensors[n["dq_norm"]]), rt.place(tensors[n["dkv_norm"]])
        if qn.dtype != cn.dtype:
            qn, cn = qn.to(torch.float32), cn.to(torch.float32)
        self.w_q_norm, self.w_c_norm = qn, cn
        if self.position is not None:
            self.position.bind(tensors, rt)

    def forward(self, h, residual, step, memory) -> None:
        H, T, dt = self.n_heads, h.shape[0], self.rt.dtype
        with ops.bucket("qkv matmul"):
            down = linear(h, self.w_down, out_dtype=dt)
        with ops.bucket("rope+cache"):
            table = self.position.table(step) if self.position is not None else None
            cq = ops.latent_prepare(down, self.w_q_norm, self.w_c_norm, self.eps, table, self.rot, step.positions,
                                    step.token_slots, memory, self.q_rank, self.rank, self.rot_dim)
        with ops.bucket("qkv matmul"):
            q = linear(cq, self.w_uq, out_dtype=dt)
            qa = torch.empty((T, H * (self.rank + self.rot_dim)), dtype=dt, device=h.device)
            ops.bmm_heads(qa, self.rank + self.rot_dim, q, self.dim + self.rot_dim, self.w_uk_t, self.rank, self.dim)
        with ops.bucket("rope+cache"):
            ops.latent_query_rot(qa, q, table, self.rot, H, self.dim, self.rot_dim, self.rank)
        with ops.bucket("attention"):
            lat = torch.empty((T, H * self.rank), dtype=dt, device=h.device)
            ops.attention_latent(qa, memory, step, H, self.rank, self.rot_dim, self.scale, lat, plan=step.plan_of(self))
        with ops.bucket("out matmul"):
            att = torch.empty((T, H * self.v_dim), dtype=dt, device=h.device)
            ops.bmm_heads(att, self.v_dim, lat, self.rank, self.w_uv, self.v_dim, self.rank)
            if self.out_gate:
                att = ops.gate_mul(att, linear(h, self.w_g, out_dtype=dt), "sigmoid")
            linear(att, self.w_o, out=residual, accumulate=True)
