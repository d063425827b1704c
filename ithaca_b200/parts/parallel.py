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

``combine: "norm_sum"`` with ``out_norms`` (one tensor name per branch) and ``norm_eps``: every branch keeps its own output
product (with its bias, if it has one: ``branch_out_bias()``), and the composite's result is
sum_i c_i * rmsnorm(branch_i(x)) * w_i, each branch's result normed over the model width with a weight of its own before
the sum; one kernel adds the biases, norms and sums.  A branch that mixes its input with the input one position
earlier before projecting it cannot share the stacked input product: it sets ``reads_input`` and ``core`` is handed
the composite's input as ``x`` (its ``branch_in()`` is then empty).
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache
from ..config.spec import PartSpec
from ..weights.loader import TensorReq
from ..csrc import ops
from .base import MIXERS, POSITIONS, Runtime, as_float32, register_mixer
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
        if spec.get("combine", "sum") == "norm_sum":
            _merge(out, {name: TensorReq((spec["hidden_size"],), init="ones") for name in spec["out_norms"]})
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
        mats = [w for br in self.branches for w in br.branch_in()]
        self.in_proj = Linear(mats, runtime) if mats else None
        outs = [br.branch_out() for br in self.branches]
        self.combine = spec.get("combine", "sum")
        if self.combine not in ("sum", "norm_sum"):
            raise ValueError(f"parallel mixer: combine {self.combine!r} is not supported (sum, norm_sum)")
        if self.combine == "sum":
            if any(getattr(br, "branch_out_bias", lambda: None)() is not None for br in self.branches):
                raise ValueError("parallel mixer: output biases need combine 'norm_sum'")
            self.o = Linear([torch.cat([o.to(outs[0].dtype) for o in outs], dim=1)], runtime)
        else:
            if len(self.branches) > 4 or len(spec["out_norms"]) != len(self.branches):
                raise ValueError("parallel mixer: norm_sum takes up to four branches and one out_norms tensor for each")
            self.outs = [Linear([o], runtime) for o in outs]
            self.out_biases = [getattr(br, "branch_out_bias", lambda: None)() for br in self.branches]
            self.out_norms = [as_float32(tensors[name], runtime) for name in spec["out_norms"]]
            self.norm_eps = float(spec["norm_eps"])
        self.n_mid = sum(br.n_mid for br in self.branches)
        if (self.in_proj.out_features if self.in_proj is not None else 0) != sum(br.n_in for br in self.branches):
            raise ValueError("parallel mixer: a branch's input matrices do not add up to its n_in")
        self.runtime = runtime

    @property
    def graph_safe(self) -> bool:
        return all(getattr(br, "graph_safe", False) for br in self.branches)

    def cache_requests(self) -> List[object]:
        return [r for br in self.branches for r in br.cache_requests()]

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        p = self.in_proj(x, out_dtype=torch.float32) if self.in_proj is not None else None
        summed = self.combine == "sum"
        mid = torch.empty((x.shape[0], self.n_mid), dtype=self.runtime.act_dtype, device=x.device) if summed else None
        a = m = 0
        results = []
        for n, (br, c) in enumerate(zip(self.branches, self.scales)):
            kw = {"x": x} if getattr(br, "reads_input", False) else {}
            pin = p[:, a:a + br.n_in] if br.n_in else None
            if summed:
                br.core(pin, mid[:, m:m + br.n_mid], ctx, cache, writes_cache, c, **kw)
            else:
                own = torch.empty((x.shape[0], br.n_mid), dtype=self.runtime.act_dtype, device=x.device)
                br.core(pin, own, ctx, cache, writes_cache, 1.0, **kw)
                results.append(self.outs[n](own, out_dtype=torch.float32))
            a += br.n_in
            m += br.n_mid
        if summed:
            self.o(mid, out=residual, accumulate=accumulate)
        else:
            ops.branch_norm_sum(results, self.out_biases, self.out_norms, self.scales, residual, self.norm_eps, accumulate)


register_mixer("parallel", ParallelMixer)
