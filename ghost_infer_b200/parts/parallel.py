"""Mixers side by side: every one reads the same input, and their outputs are added with constant weights.

`params["mixers"]`: a list of {"spec": PartSpec of a registered mixer, "scale": float}.  residual += sum_i scale_i *
mixer_i(h).  A schedule entry has one cache and one per-sequence state, so at most one of the mixers may ask for a cache
and at most one for state; each gets the entry's memory and uses its own part of it.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest, StateRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .registry import lookup, register


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.subs = []
        for m in params["mixers"]:
            spec = m["spec"]
            self.subs.append((lookup("mixer", spec.kind)(spec.params, prefix), float(m.get("scale", 1.0))))
        if not self.subs:
            raise ValueError("mixers side by side: none given")
        if sum(s.cache_request() is not None for s, _ in self.subs) > 1 or sum(s.state_request() is not None for s, _ in self.subs) > 1:
            raise ValueError("mixers side by side share one schedule entry's memory: at most one may want a cache and one a state")

    @property
    def plans_on_host(self) -> bool:
        return any(s.plans_on_host for s, _ in self.subs)

    def weights(self) -> List[WeightSpec]:
        return [w for s, _ in self.subs for w in s.weights()]

    def cache_request(self) -> Optional[CacheRequest]:
        return next((r for r in (s.cache_request() for s, _ in self.subs) if r is not None), None)

    def state_request(self) -> Optional[StateRequest]:
        return next((r for r in (s.state_request() for s, _ in self.subs) if r is not None), None)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        return tuple(s.decode_plan(n_seqs, max_kv_len, sm_count, kv_lens) for s, _ in self.subs)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        for s, _ in self.subs:
            s.bind(tensors, rt)

    def forward(self, h, residual, step, memory) -> None:
        # each mixer finds its own plan where it would look for it: under its own identity
        plans = step.plan_of(self)
        saved = step.fixed_plans
        if plans is not None:
            step.fixed_plans = dict(saved or {})
            step.fixed_plans.update({id(s): p for (s, _), p in zip(self.subs, plans)})
        try:
            for s, scale in self.subs:
                y = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
                s.forward(h, y, step, memory)
                ops.axpy(residual, y, scale)
        finally:
            step.fixed_plans = saved
