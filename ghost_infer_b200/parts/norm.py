"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in 32-bit.

eps sits inside the square root and the weight multiplies last, with no bias and no "+1"
(src/model.rs:919-928, src/cuda.rs:505-515).

"layernorm": y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w, with a weight and no bias, also 32-bit.

`forward(x, rows=None, out_dtype=None)`: `out_dtype` None is the step's activation type; a model that norms its
embeddings asks for float32, the stream's own type.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Norm, WeightSpec
from .registry import register


@register("norm", "rmsnorm")
class RmsNorm(Norm):
    settles_pending = True      # its kernel adds partial sums a deferred product left for the rows it reads

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])

    def weights(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor_name("weight", "weight"), (self.size,), "ones")]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.weight = rt.place(tensors[self.tensor_name("weight", "weight")])
        self._weight32 = None

    @property
    def weight32(self) -> torch.Tensor:
        """The weight as 32-bit values (what joins the residual sum is 32-bit), made when first asked for."""
        if self._weight32 is None:
            self._weight32 = self.weight.to(torch.float32).contiguous()
        return self._weight32

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        with ops.bucket("norm"):
            return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows=rows)


    def add_normed(self, x: torch.Tensor, y: torch.Tensor, scale: Optional[torch.Tensor] = None,
                   cast_out: Optional[torch.Tensor] = None, zero_y: bool = False) -> None:
        """x += y / sqrt(mean(y^2) + eps) * w [* scale]: the norm on a sublayer's output, joined to the stream in one pass;
        the same pass can leave the new stream in the activation type in `cast_out` and y zeroed, for the next sublayer."""
        with ops.bucket("norm"):
            ops.postnorm_add(x, y, self.weight32, self.eps, scale, cast_out=cast_out, zero_y=zero_y)


@register("norm", "channel_scale")
class ChannelScale(Norm):
    """A learned number per channel that multiplies a sublayer's normed output (kept 32-bit: it joins the residual sum)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.size = int(params["size"])

    def weights(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor_name("weight", "weight"), (self.size,), "ones")]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.weight = tensors[self.tensor_name("weight", "weight")].to(device=rt.device, dtype=torch.float32).contiguous()

    def forward(self, x, rows=None, out_dtype=None):
        raise NotImplementedError("a channel scale is applied by the block that holds it")


@register("norm", "layernorm")
class LayerNorm(Norm):
    settles_pending = True      # its kernel adds partial sums a deferred product left for the rows it reads

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])

    def weights(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor_name("weight", "weight"), (self.size,), "ones")]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.weight = rt.place(tensors[self.tensor_name("weight", "weight")])

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        with ops.bucket("norm"):
            return ops.layernorm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows=rows)
