"""A layer over several copies of the residual stream ("hyper-connections"), with a short convolution in front of every
sublayer and a gate on what it returns.

The stream of a token is `streams` vectors x_1 .. x_S (all equal to the embedded token before the first layer; summed before
the final norm).  A sublayer (the mixer, then the feed-forward if the layer has one) runs as

    u = sum_s a[s] x_s                          h = norm(u)
    c = h + conv(h)                             conv(h)_t = sum_j k[:, j] h_(t - taps + 1 + j), zeros before the sequence's start
    y = sublayer(c) * sigmoid(W_g h + b_g)      the gate reads h itself, before the convolution
    x_t <- sum_s M[s, t] x_s + o[t] y           every copy at once, from the old copies (M is indexed [from, to])

with a, M, o learned per sublayer.  Each option can be switched off by its parameter (`conv_taps` 0, `gate` False); with one
copy, a = M = o = 1 and both off it is the ordinary pre-norm residual layer.  The last taps - 1 inputs h of both sublayers are
part of a sequence's state (`memory.block_state`, 32-bit, zero at the start), so a prompt cut anywhere walks the same sums.
The blend, the norm, the gate's sigmoid, the mix and the sum are 32-bit.

Tensor names under the layer's prefix (q = 1 for the mixer, 2 for the feed-forward): "hc<q>.in" [S], "hc<q>.mix" [S, S],
"hc<q>.out" [S], "canon<q>" [width, taps], "rg<q>" [width, width], "rg<q>.b" [width]; `params["tensor_names"]` replaces any.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import ops
from .base import Block, Part, WeightSpec
from .linear import linear
from .registry import register


@register("feed_forward", "hyper_connection")
class HyperConnection(Part):
    """The learned numbers of one sublayer's connection to the copies of the stream, its input convolution and its gate
    (an `extra` part of the layer, named "connect1" / "connect2"; the block runs it)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.width = int(params["hidden_size"])
        self.streams = int(params["streams"])
        self.taps = int(params.get("conv_taps") or 0)
        self.gate = bool(params.get("gate", False))
        q = str(params["index"])
        d = {"in": f"hc{q}.in", "mix": f"hc{q}.mix", "out": f"hc{q}.out", "conv": f"canon{q}", "gate": f"rg{q}", "gate_bias": f"rg{q}.b"}
        self.names = {k: self.tensor_name(k, v) for k, v in d.items()}
        if self.streams < 1:
            raise ValueError("a layer needs at least one copy of the stream")

    def weights(self) -> List[WeightSpec]:
        n, S, d = self.names, self.streams, self.width
        out = [WeightSpec(n["in"], (S,), "ones"), WeightSpec(n["mix"], (S, S)), WeightSpec(n["out"], (S,), "ones")]
        if self.taps:
            out.append(WeightSpec(n["conv"], (d, self.taps)))
        if self.gate:
            out += [WeightSpec(n["gate"], (d, d)), WeightSpec(n["gate_bias"], (d,))]
        return out

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        f32 = lambda name: tensors[name].to(device=rt.device, dtype=torch.float32).contiguous()     # they join 32-bit sums
        self.blend, self.mix, self.share = f32(n["in"]), f32(n["mix"]), f32(n["out"])
        self.conv_w = rt.place(tensors[n["conv"]]) if self.taps else None
        self.w_gate = rt.place(tensors[n["gate"]]) if self.gate else None
        self.b_gate = rt.place(tensors[n["gate_bias"]]) if self.gate else None


@register("block", "hyper_connections")
class HyperConnections(Block):
    def _connections(self):
        return [self.extra.get("connect1"), self.extra.get("connect2")]

    def state_request(self) -> Optional[StateRequest]:
        c1, c2 = self._connections()
        taps = max((c.taps for c in (c1, c2) if c is not None), default=0)
        if taps <= 1:
            return None
        return StateRequest((2, (taps - 1) * c1.width), torch.float32)      # [sublayer][the last taps - 1 inputs, oldest first]

    def _sublayer(self, x, step, memory, which: int, norm, conn, run) -> None:
        dt = norm.rt.dtype
        n, d = x.shape[0], conn.width
        y = torch.empty((n, d), dtype=torch.float32, device=x.device)
        state = None
        if conn.taps > 1:
            if memory.block_state is None:
                raise RuntimeError("the input convolution was given no per-sequence state")
            state = memory.block_state[:, which]
        if conn.taps and step.is_decode and ops.hyper_read_conv_ok(d, conn.taps):
            # one token a sequence: every older input comes from the state, and the convolution rides in the reading pass
            with ops.bucket("norm"):
                h, c = ops.hyper_read(x, conn.blend, norm.weight, norm.eps, dt, zero=y, conv=(conn.conv_w, state, step))
        else:
            with ops.bucket("norm"):
                h = ops.hyper_read(x, conn.blend, norm.weight, norm.eps, dt, zero=y)
            with ops.bucket("conv"):
                c = ops.input_conv(h, conn.conv_w, state, step) if conn.taps else h
        with ops.bucket("out matmul"):
            z = linear(h, conn.w_gate, out_dtype=dt) if conn.gate else None
        run(c, y)
        with ops.bucket("norm"):
            ops.hyper_write(x, y, conn.mix, conn.share, z, conn.b_gate, h if state is not None else None, state, conn.taps, step)

    def forward(self, x, step, memory) -> None:
        if x.is_cuda:
            ops.settle(x)
        c1, c2 = self._connections()
        self._sublayer(x, step, memory, 0, self.mixer_norm, c1, lambda c, y: self.mixer.forward(c, y, step, memory))
        if self.ffn is not None:
            self._sublayer(x, step, memory, 1, self.ffn_norm, c2, lambda c, y: self.ffn.forward(c, y, step))
