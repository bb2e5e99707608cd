"""Routed feed-forward: a mixture of small gated feed-forward layers, of which every token uses a few.

Router logits z = W_r h, 32-bit; a token's experts are the `top` largest logits and their weights the softmax over
those logits alone; expert e computes W_down,e (silu(W_gate,e h) * (W_up,e h)), no biases; the token's output is the
weighted sum.  A shared expert of the same form (if the model has one) runs for every token and is added, multiplied
by sigmoid(w_sg . h), one number per token.  residual += all of it.

On the device the (token, choice) entries are sorted by expert without the host learning the counts, so a step's
launches do not depend on what the router chose and one-token steps can be recorded and replayed.  A prompt step in
bfloat16 with enough rows per expert reads the counts back (one wait per layer) and runs each expert's rows through
the tensor-core products the dense feed-forward uses, its gate and up rows interleaved for their gated epilogue.

Tensor names: prefix + "mlp.router", "mlp.e<i>.{gate,up,down}", "mlp.shared.{gate,up,down,sg}" unless
`params["tensor_names"]` replaces the stems "router", "expert" (a format with `{i}`) or "shared".

"scored_experts" is the routed layer in another form: the experts are ungated, W_down,e relu(W_up,e x)^2 (`activation`
"relu2"); a chosen expert's weight is `scores` "sigmoid": the sigmoid of its own logit, not renormalized (or "softmax":
as above); and with `weight_on` "input" the weight multiplies what the expert reads, out = sum_e expert_e(w_e h), instead
of what it returns ("output").  It has no shared expert.  Tensors: "mlp.router", "mlp.e<i>.{up,down}".
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import FeedForward, WeightSpec
from .linear import linear
from .registry import register


@register("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.ff = int(params["expert_ff"])
        self.shared_ff = int(params["shared_ff"]) if params.get("shared_ff") else None
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"a token cannot use {self.top} of {self.experts} experts")
        self.router_name = self.tensor_name("router", "mlp.router")
        self.expert_stem = self.tensor_name("expert", "mlp.e{i}.")
        self.shared_stem = self.tensor_name("shared", "mlp.shared.")

    def _expert(self, i: int, what: str) -> str:
        return self.expert_stem.format(i=i) + what

    def weights(self) -> List[WeightSpec]:
        out = [WeightSpec(self.router_name, (self.experts, self.hidden))]
        for i in range(self.experts):
            out += [WeightSpec(self._expert(i, "gate"), (self.ff, self.hidden)), WeightSpec(self._expert(i, "up"), (self.ff, self.hidden)),
                    WeightSpec(self._expert(i, "down"), (self.hidden, self.ff))]
        if self.shared_ff:
            s = self.shared_stem
            out += [WeightSpec(s + "gate", (self.shared_ff, self.hidden)), WeightSpec(s + "up", (self.shared_ff, self.hidden)),
                    WeightSpec(s + "down", (self.hidden, self.shared_ff)), WeightSpec(s + "sg", (1, self.hidden))]
        return out

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.w_router = rt.place(tensors[self.router_name])
        # [E, 2 f, d]: gate rows, then up rows; on the 16-bit path in blocks [8 gate | 8 up], as the products' gated
        # epilogue wants them (the kernels here read either layout)
        self.interleaved = rt.dtype == torch.bfloat16 and self.ff % 8 == 0 and rt.device.type == "cuda"
        gate_up = []
        for i in range(self.experts):
            g, u = tensors[self._expert(i, "gate")], tensors[self._expert(i, "up")]
            if self.interleaved:
                gate_up.append(torch.stack([g.reshape(self.ff // 8, 8, self.hidden), u.reshape(self.ff // 8, 8, self.hidden)], dim=1)
                               .reshape(2 * self.ff, self.hidden))
            else:
                gate_up.append(torch.cat([g, u], dim=0))
        self.w_gate_up = rt.place(torch.stack(gate_up))
        self.w_down = rt.place(torch.stack([tensors[self._expert(i, "down")] for i in range(self.experts)]))   # [E, d, f]
        if self.w_gate_up.dtype != self.w_down.dtype:
            self.w_gate_up, self.w_down = self.w_gate_up.float(), self.w_down.float()
        self.interleaved = self.interleaved and self.w_gate_up.dtype == torch.bfloat16
        self.w_sg = None
        if self.shared_ff:
            s = self.shared_stem
            g, u = rt.place(tensors[s + "gate"]), rt.place(tensors[s + "up"])
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            f = self.shared_ff
            self.shared_interleaved = (rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and f % 8 == 0
                                       and rt.device.type == "cuda")
            if self.shared_interleaved:
                self.w_shared_gu = torch.stack([g.view(f // 8, 8, self.hidden), u.view(f // 8, 8, self.hidden)], dim=1) \
                    .reshape(2 * f, self.hidden).contiguous()
            else:
                self.w_shared_gu = torch.cat([g, u], dim=0).contiguous()
            self.w_shared_down = rt.place(tensors[s + "down"])
            self.w_sg = rt.place(tensors[s + "sg"]).reshape(-1).to(self.w_router.dtype).contiguous()

    # rows per expert, on average, from which a prompt step takes the tensor-core products expert by expert
    ROWS_FOR_TENSOR_CORES = 96

    def _by_expert(self, h, step) -> bool:
        return (self.interleaved and not step.is_decode and h.dtype == torch.bfloat16 and self.hidden % 8 == 0
                and h.shape[0] * self.top >= self.ROWS_FOR_TENSOR_CORES * self.experts and not torch.cuda.is_current_stream_capturing())

    def _experts_one_by_one(self, h, offsets, perm):
        """The experts' outputs for a prompt step: the rows gathered in sorted order, then for every expert with rows
        the gated product and the down product over its stretch.  The host waits for the counts here."""
        rows = ops.moe_gather_rows(h, perm, self.top)
        return ops.moe_experts_by_expert(rows, self.w_gate_up, self.w_down, offsets.cpu().tolist())

    def forward(self, h, residual, step) -> None:
        with ops.bucket("router"):
            ids, wts, sgate = ops.moe_route(h, self.w_router, self.top, self.w_sg)
            offsets, perm, inv = ops.moe_plan(ids, self.experts)
        with ops.bucket("experts"):
            if self._by_expert(h, step):
                down = self._experts_one_by_one(h, offsets, perm)
            else:
                down = ops.moe_experts(h, self.w_gate_up, self.w_down, offsets, perm, self.top, self.interleaved)
        with ops.bucket("ffn matmul"):
            shared = None
            if self.shared_ff:
                if self.shared_interleaved:
                    act = ops.swiglu_interleaved(h, self.w_shared_gu)
                else:
                    act = ops.act_mul(linear(h, self.w_shared_gu, out_dtype=self.rt.dtype), "silu")
                shared = linear(act, self.w_shared_down, out_dtype=torch.float32)
            ops.settle(residual)
            ops.moe_combine(residual, down, inv, wts, shared, sgate)


@register("feed_forward", "scored_experts")
class ScoredExperts(FeedForward):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.ff = int(params["expert_ff"])
        self.activation = str(params.get("activation", "relu2"))
        self.scores = str(params.get("scores", "sigmoid"))
        self.weight_on = str(params.get("weight_on", "input"))
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"a token cannot use {self.top} of {self.experts} experts")
        if self.activation != "relu2" or self.scores not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError("scored experts: activation relu2; scores sigmoid or softmax; weight_on input or output")
        self.router_name = self.tensor_name("router", "mlp.router")
        self.expert_stem = self.tensor_name("expert", "mlp.e{i}.")

    def _expert(self, i: int, what: str) -> str:
        return self.expert_stem.format(i=i) + what

    def weights(self) -> List[WeightSpec]:
        out = [WeightSpec(self.router_name, (self.experts, self.hidden))]
        for i in range(self.experts):
            out += [WeightSpec(self._expert(i, "up"), (self.ff, self.hidden)), WeightSpec(self._expert(i, "down"), (self.hidden, self.ff))]
        return out

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.w_router = rt.place(tensors[self.router_name])
        self.w_up = rt.place(torch.stack([tensors[self._expert(i, "up")] for i in range(self.experts)]))       # [E, f, d]
        self.w_down = rt.place(torch.stack([tensors[self._expert(i, "down")] for i in range(self.experts)]))   # [E, d, f]
        if self.w_up.dtype != self.w_down.dtype:
            self.w_up, self.w_down = self.w_up.float(), self.w_down.float()

    # rows per expert, on average, from which a prompt step takes the tensor-core products expert by expert
    ROWS_FOR_TENSOR_CORES = 96

    def _by_expert(self, h, step) -> bool:
        return (not step.is_decode and h.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and self.hidden % 8 == 0
                and self.ff % 8 == 0 and h.shape[0] * self.top >= self.ROWS_FOR_TENSOR_CORES * self.experts
                and not torch.cuda.is_current_stream_capturing())

    def forward(self, h, residual, step) -> None:
        with ops.bucket("router"):
            ids, wts, _ = ops.moe_route(h, self.w_router, self.top, None, scores=self.scores)
            offsets, perm, inv = ops.moe_plan(ids, self.experts)
        with ops.bucket("experts"):
            # the rows in the order of the sort, each times its entry's weight where the weight goes onto the input
            rows = ops.moe_gather_rows(h, perm, self.top, wts.view(-1) if self.weight_on == "input" else None)
            if self._by_expert(h, step):
                # enough rows per expert: the host reads the experts' offsets back (one wait) and every expert's stretch
                # goes through the products the dense layers use
                down = ops.moe_experts_by_expert_ungated(rows, self.w_up, self.w_down, offsets.cpu().tolist())
            else:
                hidden = ops.moe_rows_product(rows, self.w_up, offsets, act=self.activation)
                down = ops.moe_rows_product(hidden, self.w_down, offsets)
        with ops.bucket("ffn matmul"):
            ops.settle(residual)
            ops.moe_combine(residual, down, inv, wts if self.weight_on == "output" else None)


@register("feed_forward", "share_routed_experts")
class ShareRoutedExperts(FeedForward):
    """Routed gated experts whose router scores every expert by its share of a softmax over ALL experts.

    z = W_r h (32-bit); s = softmax(z) over all experts; the `top` experts with the largest s + `correction` (a stored vector,
    one number per expert; it steers the choice only) are chosen; their weights are s (without the correction) divided by
    the sum of the chosen shares (+ 1e-20), times `route_scale`.  An expert, and the shared expert that runs for every token
    and is added as it is, computes W_down (g sigmoid(`alpha` g) (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h,
    -limit, limit) (`limit` for the routed experts, `shared_limit` for the shared one; 0 or None: no clamps).  No biases.

    Tensors: "mlp.router", "mlp.correction", "mlp.e<i>.{gate,up,down}", "mlp.shared.{gate,up,down}" unless
    `params["tensor_names"]` replaces the stems "router", "correction", "expert" (a format with `{i}`) or "shared"."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.ff = int(params["expert_ff"])
        self.limit = float(params.get("limit") or 0.0)
        self.alpha = float(params.get("alpha", 1.0))
        self.route_scale = float(params.get("route_scale", 1.0))
        self.has_correction = bool(params.get("correction", True))
        self.shared_ff = int(params["shared_ff"]) if params.get("shared_ff") else None
        self.shared_limit = float(params.get("shared_limit") or 0.0)
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"a token cannot use {self.top} of {self.experts} experts")
        self.router_name = self.tensor_name("router", "mlp.router")
        self.correction_name = self.tensor_name("correction", "mlp.correction")
        self.expert_stem = self.tensor_name("expert", "mlp.e{i}.")
        self.shared_stem = self.tensor_name("shared", "mlp.shared.")

    def _expert(self, i: int, what: str) -> str:
        return self.expert_stem.format(i=i) + what

    def weights(self) -> List[WeightSpec]:
        out = [WeightSpec(self.router_name, (self.experts, self.hidden))]
        if self.has_correction:
            out.append(WeightSpec(self.correction_name, (self.experts,)))
        for i in range(self.experts):
            out += [WeightSpec(self._expert(i, "gate"), (self.ff, self.hidden)), WeightSpec(self._expert(i, "up"), (self.ff, self.hidden)),
                    WeightSpec(self._expert(i, "down"), (self.hidden, self.ff))]
        if self.shared_ff:
            s = self.shared_stem
            out += [WeightSpec(s + "gate", (self.shared_ff, self.hidden)), WeightSpec(s + "up", (self.shared_ff, self.hidden)),
                    WeightSpec(s + "down", (self.hidden, self.shared_ff))]
        return out

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.w_router = rt.place(tensors[self.router_name])
        # the correction joins 32-bit shares: kept as 32-bit values
        self.correction = (tensors[self.correction_name].to(device=rt.device, dtype=torch.float32).contiguous()
                           if self.has_correction else None)
        # [E, 2 f, d]: gate rows, then up rows; on the 16-bit path in blocks [8 gate | 8 up], as the tensor-core product's gated
        # epilogue wants them (the plain kernels read either layout)
        self.interleaved = rt.dtype == torch.bfloat16 and self.ff % 8 == 0 and rt.device.type == "cuda"
        gate_up = []
        for i in range(self.experts):
            g, u = tensors[self._expert(i, "gate")], tensors[self._expert(i, "up")]
            if self.interleaved:
                gate_up.append(torch.stack([g.reshape(self.ff // 8, 8, self.hidden), u.reshape(self.ff // 8, 8, self.hidden)], dim=1)
                               .reshape(2 * self.ff, self.hidden))
            else:
                gate_up.append(torch.cat([g, u], dim=0))
        self.w_gate_up = rt.place(torch.stack(gate_up))
        self.w_down = rt.place(torch.stack([tensors[self._expert(i, "down")] for i in range(self.experts)]))   # [E, d, f]
        if self.w_gate_up.dtype != self.w_down.dtype:
            self.w_gate_up, self.w_down = self.w_gate_up.float(), self.w_down.float()
        self.interleaved = self.interleaved and self.w_gate_up.dtype == torch.bfloat16
        if self.shared_ff:
            s = self.shared_stem
            g, u = rt.place(tensors[s + "gate"]), rt.place(tensors[s + "up"])
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            f = self.shared_ff
            # 16-bit path: gate and up rows in blocks of 8, so that the products' gated epilogues hold both halves of a value
            self.shared_interleaved = (rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and f % 8 == 0 and rt.device.type == "cuda")
            if self.shared_interleaved:
                self.w_shared_gu = torch.stack([g.view(f // 8, 8, self.hidden), u.view(f // 8, 8, self.hidden)], dim=1) \
                    .reshape(2 * f, self.hidden).contiguous()
            else:
                self.w_shared_gu = torch.cat([g, u], dim=0).contiguous()
            self.w_shared_down = rt.place(tensors[s + "down"])

    # rows per expert, on average, from which a prompt step takes the tensor-core products expert by expert
    ROWS_FOR_TENSOR_CORES = 96

    def _by_expert(self, h, step) -> bool:
        return (self.interleaved and self.limit > 0 and not step.is_decode and h.dtype == torch.bfloat16 and self.hidden % 8 == 0
                and h.shape[0] * self.top >= self.ROWS_FOR_TENSOR_CORES * self.experts and not torch.cuda.is_current_stream_capturing())

    def forward(self, h, residual, step) -> None:
        with ops.bucket("router"):
            ids, wts = ops.moe_route_shares(h, self.w_router, self.top, self.correction, self.route_scale)
            offsets, perm, inv = ops.moe_plan(ids, self.experts)
        with ops.bucket("experts"):
            if self._by_expert(h, step):
                # enough rows per expert: the host reads the experts' offsets back (one wait) and every expert's stretch goes
                # through the products the dense layers use, the clamped gate in the first one's epilogue
                rows = ops.moe_gather_rows(h, perm, self.top)
                down = ops.moe_experts_by_expert(rows, self.w_gate_up, self.w_down, offsets.cpu().tolist(), self.limit, self.alpha)
            else:
                down = ops.moe_experts(h, self.w_gate_up, self.w_down, offsets, perm, self.top, self.interleaved, self.limit, self.alpha)
        with ops.bucket("ffn matmul"):
            ops.settle(residual)
            if self.shared_ff:
                if self.shared_interleaved:
                    act = ops.clamped_glu_interleaved(h, self.w_shared_gu, self.shared_limit, self.alpha)
                else:
                    act = ops.clamped_glu(linear(h, self.w_shared_gu, out_dtype=self.rt.dtype), self.shared_limit, self.alpha)
                linear(act, self.w_shared_down, out=residual, accumulate=True)
            ops.moe_combine(residual, down, inv, wts)
