"""A mixer made of several mixers side by side: y = sum_i c_i * branch_i(x), all reading the same input.

``branches`` is a list of part records (kind, sizes, tensor names; a branch that takes positions carries its
position record under ``position``), ``scales`` the constants c_i.  A branch class offers, beside the usual
interface, ``branch_in()`` (the matrices that multiply the input, in the order of the columns its ``core`` reads),
``branch_out()`` (the matrix that multiplies what ``core`` writes), ``n_in`` / ``n_mid`` (those widths) and
``core(p, mid, ctx, cache, writes_cache, mult)``.  The composite stacks all branches' input matrices into ONE product
and all output matrices, side by side along their input dimension, into ONE product: the branches' results, each
already multiplied by its constant, lie next to each other in one operand, and the sum over branches happens inside
the output product's accumulation.  Every branch keeps what it needs in the same cache entry (keys and values for one,
a fixed-size state for another).
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache
from ..config.spec import PartSpec
from ..weights.loader import TensorReq
from .base import MIXERS, POSITIONS, Runtime, register_mixer
from .linear import Linear


def _merge(into: Dict[str, TensorReq], more: Mapping[str, TensorReq]) -> None:
    for name, req in more.items():
        if name in into:
            raise ValueError(f"tensor '{name}' is asked for by two branches")
        into[name] = req


class ParallelMixer:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for b in spec["branches"]:
            _merge(out, MIXERS.get(b.kind).manifest(b))
            pos = b.get("position")
            if pos is not None:
                _merge(out, POSITIONS.get(pos.kind).manifest(pos))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.scales = [float(c) for c in spec["scales"]]
        if len(self.scales) != len(spec["branches"]) or not self.scales:
            raise ValueError("parallel mixer: one constant per branch is needed")
        self.branches = []
        for b in spec["branches"]:
            cls_ = MIXERS.get(b.kind)
            params = inspect.signature(cls_.__init__).parameters
            if "standalone" not in params or not hasattr(cls_, "core"):
                raise ValueError(f"parallel mixer: mixer kind '{b.kind}' cannot serve as a branch")
            kw = {"standalone": False}
            pos = b.get("position")
            if pos is not None:
                if "position" not in params:
                    raise ValueError(f"parallel mixer: mixer kind '{b.kind}' takes no positions")
                kw["position"] = POSITIONS.get(pos.kind)(pos, tensors, runtime)
            self.branches.append(cls_(b, tensors, runtime, **kw))
        self.in_proj = Linear([w for br in self.branches for w in br.branch_in()], runtime)
        outs = [br.branch_out() for br in self.branches]
        self.o = Linear([torch.cat([o.to(outs[0].dtype) for o in outs], dim=1)], runtime)
        self.n_mid = sum(br.n_mid for br in self.branches)
        if self.in_proj.out_features != sum(br.n_in for br in self.branches):
            raise ValueError("parallel mixer: a branch's input matrices do not add up to its n_in")
        self.runtime = runtime

    @property
    def graph_safe(self) -> bool:
        return all(getattr(br, "graph_safe", False) for br in self.branches)

    def cache_requests(self) -> List[object]:
        return [r for br in self.branches for r in br.cache_requests()]

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        p = self.in_proj(x, out_dtype=torch.float32)
        mid = torch.empty((x.shape[0], self.n_mid), dtype=self.runtime.act_dtype, device=x.device)
        a = m = 0
        for br, c in zip(self.branches, self.scales):
            br.core(p[:, a:a + br.n_in], mid[:, m:m + br.n_mid], ctx, cache, writes_cache, c)
            a += br.n_in
            m += br.n_mid
        self.o(mid, out=residual, accumulate=accumulate)


register_mixer("parallel", ParallelMixer)
