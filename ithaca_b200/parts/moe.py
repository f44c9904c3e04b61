"""Mixture of experts: a router and small gated feed-forwards, of which each token uses a few.

Router: z = Wr x in float32 (x may be the activations' 16-bit rounding), scores = softmax(z)
over all experts.  Experts may form equal groups of neighbours: a group counts by its best
score, and only experts of the ``group_keep`` best groups can be chosen.  The ``top`` best of
them are; their weights are their scores (``renormalize``: divided by their sum).  An expert is
y = Wd (silu(Wg x) * (Wu x)); the layer's output is the weighted sum of the chosen experts'.

On the device: one kernel picks experts and weights per token; a counting sort groups the
(token, choice) pairs by expert; two grouped products run every expert over its rows (the first
with silu(g) * u as its epilogue, so the [rows, 2 ff] intermediate is never written); a last kernel
adds a token's choices in the order they were chosen.  Nothing is read back by the host: grids are
sized from upper bounds, so a captured step can be replayed.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, register_feed_forward, to_device


class MoEFeedForward:
    graph_safe = True

    @classmethod
    def _roles(cls, spec: PartSpec):
        """The spec names the router's tensor and a pattern per expert matrix with ``{e}`` for the expert."""
        w = spec.weights
        E = int(spec["n_experts"])
        return w["router"], [(w["gate"].format(e=e), w["up"].format(e=e), w["down"].format(e=e)) for e in range(E)]

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, ff = spec["hidden_size"], spec["intermediate_size"]
        router, experts = cls._roles(spec)
        out = {router: TensorReq((spec["n_experts"], d), std=2.0 / d ** 0.5)}       # random weights: logits a few units apart
        for g, u, dn in experts:
            out[g], out[u], out[dn] = TensorReq((ff, d)), TensorReq((ff, d)), TensorReq((d, ff))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        act = spec.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"moe: activation {act!r} is not supported (silu)")
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        self.n_experts = int(spec["n_experts"])
        self.top = int(spec["top"])
        self.n_groups = int(spec.get("n_groups") or 0)
        self.group_keep = int(spec.get("group_keep") or 0)
        self.renormalize = bool(spec.get("renormalize", False))
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"moe: top must lie in 1..{self.n_experts}, found {self.top}")
        if self.n_groups > 1:
            if self.n_experts % self.n_groups or not 1 <= self.group_keep <= self.n_groups:
                raise ValueError(f"moe: {self.n_experts} experts do not form {self.n_groups} equal groups of which "
                                 f"{self.group_keep} are kept")
            if self.top > self.group_keep * (self.n_experts // self.n_groups):
                raise ValueError("moe: the kept groups hold fewer experts than a token is to use")
        router, experts = self._roles(spec)
        wt = torch.bfloat16 if runtime.dtype == "bfloat16" else None
        # the router stays float32 whatever the path: its products are formed and added in 32 bits
        self.router = to_device(tensors[router], runtime).to(torch.float32).contiguous()

        def stack(mats):
            t = torch.stack([to_device(m, runtime) for m in mats], dim=0)
            return (t.to(wt) if wt is not None else t).contiguous()

        self.gate_up = stack([torch.cat((tensors[g], tensors[u]), dim=0) for g, u, _ in experts])     # [E, 2 ff, d]
        self.down = stack([tensors[dn] for _, _, dn in experts])                                       # [E, d, ff]
        self.runtime = runtime

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, accumulate: bool = True) -> None:
        rt = self.runtime
        logits = ops.gemm_simt(x, self.router, out_dtype=torch.float32)
        chosen, weight = ops.moe_route(logits, self.top, self.n_groups, self.group_keep, self.renormalize)
        plan = ops.moe_sort(chosen, self.n_experts)
        h = ops.moe_gemm(0, x, self.gate_up, plan, rt.act_dtype)
        parts = ops.moe_gemm(1, h, self.down, plan, torch.float32)
        if accumulate:
            ops.add_(residual, ops.moe_combine(parts, weight))
        else:
            ops.moe_combine(parts, weight, out=residual)


register_feed_forward("moe", MoEFeedForward)
