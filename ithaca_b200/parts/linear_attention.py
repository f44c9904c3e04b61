"""Linear attention with one constant decay per head ("lightning attention").

Per head h with decay a_h in (0, 1]:  S_t = a_h S_(t-1) + k_t v_t^T  (S is head_dim x v_head_dim, zero before the
sequence's first token),  o_t = S_t^T q_t.  q, k and v are projections of the mixer's input passed through an
activation (``silu``; ``none``); no score scale, no softmax, no positions.  The heads' results together are RMS-normed
with a weight (``norm_eps`` inside the root), optionally multiplied by sigmoid of a full-width projection of the
input (``gate``), and projected out.

The state is float32 [2, heads, head_dim, v_head_dim] per sequence and cache entry: two copies by the parity of
the position the state belongs to, so that a decode step never overwrites the state it read (a step that is run
twice, as graph capture does, leaves the same state).  The recurrence, its decays and sums are float32 on both
paths; only the projections' operands are 16-bit on the bfloat16 path.

Like the wide attention, the mixer can serve as a branch of a composite (``parts/parallel.py``).
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_mixer
from .linear import Linear

STATE = "decay_state"


class DecayAttention:
    graph_safe = True       # slots, positions and lengths come from device arrays; the state is kept by parity

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, H, dk, dv = spec["hidden_size"], spec["n_heads"], spec["head_dim"], spec["v_head_dim"]
        w = spec.weights
        out = {w["q"]: TensorReq((H * dk, d)), w["k"]: TensorReq((H * dk, d)), w["v"]: TensorReq((H * dv, d)),
               w["o"]: TensorReq((d, H * dv)), w["norm"]: TensorReq((H * dv,), init="ones")}
        if spec.get("gate"):
            out[w["g"]] = TensorReq((H * dv, d))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, standalone: bool = True):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_head_dim = int(spec["v_head_dim"])
        if self.head_dim > 256:
            raise ValueError(f"decay_attention: the kernels hold a head's key rows in registers, up to 256 of them; found {self.head_dim}")
        decay = [float(a) for a in spec["decay"]]
        if len(decay) != self.n_heads:
            raise ValueError(f"decay_attention: {len(decay)} decays for {self.n_heads} heads")
        act = spec.get("activation", "silu")
        if act not in ("silu", "none"):
            raise ValueError(f"decay_attention: activation {act!r} is not supported (silu, none)")
        # 0 none, 1 silu, 2 silu with the hardware's approximate exponential (what feeds 16-bit products anyway)
        self.act = 0 if act == "none" else 2 if runtime.dtype == "bfloat16" else 1
        self.gate = bool(spec.get("gate"))
        self.norm_eps = float(spec["norm_eps"])
        self.decay = torch.tensor(decay, dtype=torch.float32, device=runtime.device)
        w = spec.weights
        self.norm_w = as_float32(tensors[w["norm"]], runtime)
        self._in = [tensors[w["q"]], tensors[w["k"]], tensors[w["v"]]] + ([tensors[w["g"]]] if self.gate else [])
        self._out = tensors[w["o"]]
        self.k_off = self.n_heads * self.head_dim
        self.v_off = 2 * self.k_off
        self.g_off = self.v_off + self.n_heads * self.v_head_dim
        self.n_mid = self.n_heads * self.v_head_dim
        self.n_in = self.g_off + (self.n_mid if self.gate else 0)
        if standalone:
            self.in_proj = Linear(self._in, runtime)
            self.o = Linear([self._out], runtime)
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        return [StateRequest(STATE, (2, self.n_heads, self.head_dim, self.v_head_dim), "float32")]

    def branch_in(self):
        return list(self._in)

    def branch_out(self):
        return self._out

    def core(self, p: torch.Tensor, mid: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True, mult: float = 1.0) -> None:
        """``p`` [T, n_in] float: [q | k | v | g]; ``mid`` [T, n_mid] receives ``mult`` times the normed, gated heads."""
        if not writes_cache:
            raise ValueError("decay_attention: a run cannot read another run's state without advancing it")
        o = ops.decay_attention(p, 0, self.k_off, self.v_off, self.decay, cache.state(STATE), ctx, self.n_heads, self.head_dim,
                                self.v_head_dim, self.act)
        ops.gated_rmsnorm(o, self.norm_w, self.norm_eps, p if self.gate else None, self.g_off, mid, mult)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        p = self.in_proj(x, out_dtype=torch.float32)
        mid = torch.empty((x.shape[0], self.n_mid), dtype=self.runtime.act_dtype, device=x.device)
        self.core(p, mid, ctx, cache, writes_cache)
        self.o(mid, out=residual, accumulate=accumulate)


register_mixer("decay_attention", DecayAttention)
