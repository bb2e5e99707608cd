"""A per-layer input from the token itself, added to the stream after a layer's sublayers.

With x the stream and e the layer's slice [col0, col0 + dim) of a second embedding table's row for the token:
g = gelu_tanh(W_gate x) * e;  y = W_proj g;  x += y / sqrt(mean(y^2) + eps) * w.  The table is one tensor for all layers
(`params["table"]`, a full tensor name; every layer's part names it, it is loaded once).  Norm and sum are 32-bit.

Tensor names: prefix + "side.{gate,proj,norm}" unless `params["tensor_names"]` gives others.
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import FeedForward, WeightSpec
from .linear import linear
from .registry import register


@register("feed_forward", "token_side")
class TokenSide(FeedForward):
    reads_stream = True        # its input is the stream itself, not a normed copy

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.dim = int(params["dim"])
        self.col0 = int(params["col0"])
        self.table_width = int(params["table_width"])
        self.vocab = int(params["vocab_size"])
        self.eps = float(params["eps"])
        self.table_name = str(params["table"])
        if self.col0 < 0 or self.col0 + self.dim > self.table_width:
            raise ValueError(f"columns {self.col0}..{self.col0 + self.dim} are outside a table {self.table_width} wide")
        self.names = {k: self.tensor_name(k, f"side.{k}") for k in ("gate", "proj", "norm")}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(self.table_name, (self.vocab, self.table_width), "normal", True),
                WeightSpec(n["gate"], (self.dim, self.hidden)), WeightSpec(n["proj"], (self.hidden, self.dim)),
                WeightSpec(n["norm"], (self.hidden,), "ones")]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.table = rt.place_shared(self.table_name, tensors[self.table_name])
        self.w_gate, self.w_proj = rt.place(tensors[self.names["gate"]]), rt.place(tensors[self.names["proj"]])
        self.norm_w = tensors[self.names["norm"]].to(device=rt.device, dtype=torch.float32).contiguous()

    def forward(self, h, residual, step) -> None:
        with ops.bucket("ffn matmul"):
            gx = linear(h, self.w_gate, out_dtype=self.rt.dtype)
            g = ops.side_gate(gx, self.table, step.tokens, self.col0, self.dim)
            y = linear(g, self.w_proj, out_dtype=torch.float32)
        with ops.bucket("norm"):
            ops.postnorm_add(residual, y, self.norm_w, self.eps)
