"""The selective scan mixer ("mamba1").

[u | z] = W_in x (``inner`` channels each).  u passes a causal convolution over time per channel (``conv_taps`` taps,
with bias; the last column of the stored [channels, taps] matrix meets the current token, zeros stand before the
sequence's start) and silu.  [r | B | C] = W_x u with ``dt_rank``, ``state`` and ``state`` columns.  The step size is
dt = softplus(W_dt r + bias), one per channel; A = -exp(A_log), [inner, state].  Per channel c and state n:

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;    y_c = sum_n S[c, n] C_n + D_c u_c

and the mixer's result is W_o (y * silu(z)).

Per sequence and cache entry the mixer keeps S as float32 [2, inner, state] (two copies by the parity of the position
the state belongs to, so that a decode step never overwrites what it read) and a ring of the last ``conv_taps`` inputs
of the convolution, float32.  The step sizes, softplus, exponentials, the state and its sums are float32 on both
paths; the projections' operands and the convolution's output are 16-bit on the bfloat16 path.
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_mixer, to_device
from .linear import Linear

STATE, RING = "scan_state", "scan_conv_ring"


class SelectiveScan:
    graph_safe = True       # slots, positions and lengths come from device arrays; state by parity, ring by position

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, inner, N, R, taps = spec["hidden_size"], spec["inner"], spec["state"], spec["dt_rank"], spec["conv_taps"]
        w = spec.weights
        return {w["in"]: TensorReq((2 * inner, d)), w["conv"]: TensorReq((inner, taps), std=1.0 / taps),
                w["conv_bias"]: TensorReq((inner,)), w["x"]: TensorReq((R + 2 * N, inner)),
                w["dt"]: TensorReq((inner, R), std=R ** -0.5), w["dt_bias"]: TensorReq((inner,), std=0.5),
                w["A_log"]: TensorReq((inner, N), std=0.5), w["D"]: TensorReq((inner,), init="ones"),
                w["o"]: TensorReq((d, inner))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.hidden = int(spec["hidden_size"])
        self.inner = int(spec["inner"])
        self.n_state = int(spec["state"])
        self.dt_rank = int(spec["dt_rank"])
        self.taps = int(spec["conv_taps"])
        if self.n_state > 256:
            raise ValueError(f"mamba1: the kernels hold a channel's states in one warp's registers, up to 256 of them; found {self.n_state}")
        w = spec.weights
        self.in_proj = Linear([tensors[w["in"]]], runtime)
        self.x_proj = Linear([tensors[w["x"]]], runtime)
        self.dt_proj = Linear([tensors[w["dt"]]], runtime)
        self.o = Linear([tensors[w["o"]]], runtime)
        self.conv_w = to_device(tensors[w["conv"]], runtime).to(torch.float32).t().contiguous()      # tap-major [taps, inner]
        self.conv_b = as_float32(tensors[w["conv_bias"]], runtime)
        self.dt_bias = as_float32(tensors[w["dt_bias"]], runtime)
        self.A = (-torch.exp(as_float32(tensors[w["A_log"]], runtime))).contiguous()
        self.D = as_float32(tensors[w["D"]], runtime)
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        out: List[object] = [StateRequest(STATE, (2, self.inner, self.n_state), "float32")]
        if self.taps > 1:
            out.append(StateRequest(RING, (self.taps, self.inner), "float32"))
        return out

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        if not writes_cache:
            raise ValueError("mamba1: a run cannot read another run's state without advancing it")
        rt, inner, N, R = self.runtime, self.inner, self.n_state, self.dt_rank
        uz = self.in_proj(x, out_dtype=torch.float32)                                  # [T, 2 inner]: u then z
        ring = cache.state(RING) if self.taps > 1 else None
        u = ops.causal_conv(uz[:, :inner], self.conv_w, self.conv_b, ring, ctx, rt.act_dtype, act=True)
        rbc = self.x_proj(u, out_dtype=torch.float32)                                  # [T, R + 2 N]: r, B, C
        r = rbc[:, :R] if rt.act_dtype == torch.float32 else ops.cast(rbc[:, :R], rt.act_dtype)
        dt_raw = self.dt_proj(r, out_dtype=torch.float32)
        y = ops.selective_scan(u, dt_raw, self.dt_bias, self.A, rbc, R, R + N, self.D, uz[:, inner:], cache.state(STATE), ctx,
                               rt.act_dtype)
        self.o(y, out=residual, accumulate=accumulate)


register_mixer("mamba1", SelectiveScan)
