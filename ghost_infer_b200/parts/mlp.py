"""SwiGLU feed-forward: residual += Wdown (silu(Wgate h) * (Wup h)), silu(g) = g / (1 + exp(-g)).

No biases; gate and up are one product over the two matrices stacked by rows, as the reference's GPU
path packs them (src/quant.rs:1135-1154, src/model.rs:1133-1147, src/cuda.rs:9238-9256).

Tensor names: prefix + "mlp.{gate,up,down}_proj.weight" unless `params["tensor_names"]` gives others for the
keys "gate", "up", "down".

The same layer with another activation in place of silu (`params["activation"]`: "silu", the default, or
"gelu_tanh", 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))) is registered as "gated_mlp".

"mlp": the ungated layer residual += Wdown act(Wup h + b_up) + b_down, with `activation` "relu2" (relu(z)^2) or "gelu"
(0.5 z (1 + erf(z / sqrt 2)), without biases) and, with
`bias` (the default), a bias on both products.  Tensor names: prefix + "mlp.{up,down}" and the same + ".b" for the biases,
unless `params["tensor_names"]` gives others for the keys "up", "up_bias", "down", "down_bias".
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import FeedForward, WeightSpec
from .linear import linear
from .registry import register


@register("feed_forward", "gated_mlp")
@register("feed_forward", "swiglu")
class SwiGlu(FeedForward):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"unknown activation \"{self.activation}\" (silu, gelu_tanh)")
        self.names = {k: self.tensor_name(k, f"mlp.{k}_proj.weight") for k in ("gate", "up", "down")}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["gate"], (self.inter, self.hidden)), WeightSpec(n["up"], (self.inter, self.hidden)),
                WeightSpec(n["down"], (self.hidden, self.inter))]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        g, u = rt.place(tensors[self.names["gate"]]), rt.place(tensors[self.names["up"]])
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # 16-bit path: gate and up rows interleaved in blocks of 8, so that one block of the decode kernel
        # holds both halves of an activation and applies SwiGLU before anything is written
        self.interleaved = (rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and self.inter % 8 == 0
                            and rt.device.type == "cuda")
        if self.interleaved:
            blocks = self.inter // 8
            self.w_gate_up = torch.stack([g.view(blocks, 8, self.hidden), u.view(blocks, 8, self.hidden)], dim=1) \
                .reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        del g, u
        self.w_down = rt.place(tensors[self.names["down"]])

    def forward(self, h, residual, step) -> None:
        with ops.bucket("ffn matmul"):
            if self.interleaved:
                act = ops.swiglu_interleaved(h, self.w_gate_up, self.activation)
            else:
                gu = linear(h, self.w_gate_up, out_dtype=self.rt.dtype)
                act = ops.silu_mul(gu) if self.activation == "silu" else ops.act_mul(gu, self.activation)
            linear(act, self.w_down, out=residual, accumulate=True)


@register("feed_forward", "mlp")
class Mlp(FeedForward):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "relu2"))
        self.bias = bool(params.get("bias", True))
        if self.activation not in ("relu2", "gelu"):
            raise ValueError(f"unknown activation \"{self.activation}\" (relu2, gelu)")
        if self.activation == "gelu" and self.bias:
            raise ValueError("the gelu layer has no biases")
        d = {"up": "mlp.up", "up_bias": "mlp.up.b", "down": "mlp.down", "down_bias": "mlp.down.b"}
        self.names = {k: self.tensor_name(k, v) for k, v in d.items()}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        out = [WeightSpec(n["up"], (self.inter, self.hidden)), WeightSpec(n["down"], (self.hidden, self.inter))]
        if self.bias:
            out += [WeightSpec(n["up_bias"], (self.inter,)), WeightSpec(n["down_bias"], (self.hidden,))]
        return out

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.w_up, self.w_down = rt.place(tensors[self.names["up"]]), rt.place(tensors[self.names["down"]])
        self.b_up = self.b_down = None
        if self.bias:
            bu, bd = rt.place(tensors[self.names["up_bias"]]), rt.place(tensors[self.names["down_bias"]])
            if bu.dtype != bd.dtype:
                bu, bd = bu.to(torch.float32), bd.to(torch.float32)
            self.b_up, self.b_down = bu, bd

    def forward(self, h, residual, step) -> None:
        if self.activation == "gelu":           # the exact (erf) form: in a prompt step's product, else a step of its own
            with ops.bucket("ffn matmul"):
                act = ops.linear_act(h, self.w_up, None, "gelu")
                linear(act, self.w_down, out=residual, accumulate=True)
            return
        with ops.bucket("ffn matmul"):
            if self.bias:
                ops.settle(residual)         # the rows get the output's bias from a plain kernel, which adds no partial sums
            if step.is_decode or not h.is_cuda or h.dtype != torch.bfloat16:
                # bias and activation as a step of its own, which also puts the output's bias onto the stream
                up = linear(h, self.w_up, out_dtype=self.rt.dtype)
                act = ops.bias_act(up, self.b_up, self.activation, residual if self.bias else None, self.b_down)
            else:
                act = ops.linear_act(h, self.w_up, self.b_up, self.activation)      # in the product's epilogue where it can
                if self.bias:
                    ops.add_row_bias(residual, self.b_down)
            linear(act, self.w_down, out=residual, accumulate=True)
