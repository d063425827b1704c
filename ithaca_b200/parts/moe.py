"""Mixture of experts: a router and small feed-forwards, of which each token uses a few.

Router: z = Wr x in float32 (x may be the activations' 16-bit rounding), scores = softmax(z)
over all experts (``score: "sigmoid"``: the sigmoid of every logit by itself).  Experts may form equal groups of neighbours: a group counts by its best
score, and only experts of the ``group_keep`` best groups can be chosen.  The ``top`` best of
them are; their weights are their scores (``renormalize``: divided by their sum).  An expert is
y = Wd (silu(Wg x) * (Wu x)); the layer's output is the weighted sum of the chosen experts'.

``expert: "plain"``: an expert is ungated, y = Wd act(Wu x) with ``activation`` ``relu2`` or ``gelu_tanh`` (no ``gate`` tensors).
``weight_on: "input"``: the weight multiplies what the expert reads instead of what it gives, y = sum_e expert_e(w_e x); the
scaled rows are formed (in float, rounded once to the operands' type) while the tokens are gathered into expert order.

On the device: one kernel forms the router's logits and picks experts and weights per token; a counting sort groups the
(token, choice) pairs by expert; two grouped products run every expert over its rows (the first
with silu(g) * u as its epilogue, so the [rows, 2 ff] intermediate is never written); a last kernel
adds a token's choices in the order they were chosen.  Nothing is read back by the host: grids are
sized from upper bounds, so a captured step can be replayed.

The bfloat16 path's products are the tcgen05 product in its grouped mode: the pairs are laid out so
that every expert's rows start at a multiple of the token tile's height, the tokens' activations are
gathered into that order, and each token tile multiplies its expert's slice of the stacked weights.
The tile height follows the rows an expert gets on average (16 for a decode step, up to 256 for a
long prompt).  The float32 path, and sizes the tensor-core kernel does not take (widths that are no
multiple of 8), run the CUDA-core grouped product.
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
        gated = spec.get("expert", "gated") != "plain"
        return w["router"], [(w["gate"].format(e=e) if gated else None, w["up"].format(e=e), w["down"].format(e=e)) for e in range(E)]

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, ff = spec["hidden_size"], spec["intermediate_size"]
        router, experts = cls._roles(spec)
        out = {router: TensorReq((spec["n_experts"], d), std=2.0 / d ** 0.5)}       # random weights: logits a few units apart
        for g, u, dn in experts:
            out[u], out[dn] = TensorReq((ff, d)), TensorReq((d, ff))
            if g is not None:
                out[g] = TensorReq((ff, d))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        kind = spec.get("expert", "gated")
        if kind not in ("gated", "plain"):
            raise ValueError(f"moe: expert {kind!r} is not supported (gated, plain)")
        self.gated = kind == "gated"
        act = spec.get("activation", "silu" if self.gated else "relu2")
        if self.gated and act != "silu":
            raise ValueError(f"moe: activation {act!r} is not supported by gated experts (silu)")
        if not self.gated and act not in ops.PLAIN_ACTS:
            raise ValueError(f"moe: activation {act!r} is not supported by plain experts ({', '.join(ops.PLAIN_ACTS)})")
        self.act = act
        self.score = spec.get("score", "softmax")
        if self.score not in ops.MOE_SCORES:
            raise ValueError(f"moe: score {self.score!r} is not supported ({', '.join(ops.MOE_SCORES)})")
        where = spec.get("weight_on", "output")
        if where not in ("output", "input"):
            raise ValueError(f"moe: weight_on {where!r} is not supported (output, input)")
        self.weight_on_input = where == "input"
        if self.weight_on_input and self.gated:
            raise ValueError("moe: weights on the experts' input are built for plain experts only")
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

        # gate j and up j in rows 2j and 2j + 1, so that a product tile holds both halves of every pair it covers
        if self.gated:
            self.gate_up = stack([torch.stack((tensors[g], tensors[u]), dim=1).reshape(2 * self.intermediate, self.hidden)
                                  for g, u, _ in experts])                                             # [E, 2 ff, d]
        else:
            self.up = stack([tensors[u] for _, u, _ in experts])                                       # [E, ff, d]
        self.down = stack([tensors[dn] for _, _, dn in experts])                                       # [E, d, ff]
        self.runtime = runtime
        self.tensor_cores = runtime.dtype == "bfloat16" and self.hidden % 8 == 0 and self.intermediate % 8 == 0

    def tile_rows(self, n_tokens: int) -> int:
        """Height of a token tile of the grouped tensor-core products: about the rows an expert gets on average."""
        per = -(-n_tokens * self.top // self.n_experts)
        return 256 if per >= 1024 else 128 if per > 64 else max(16, -(-per // 16) * 16)

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, accumulate: bool = True) -> None:
        rt = self.runtime
        routed = ops.moe_router(x, self.router, self.top, self.n_groups, self.group_keep, self.renormalize, self.score)
        if routed is None:                                   # sizes beyond the fused kernel's shared memory
            logits = ops.gemm_simt(x, self.router, out_dtype=torch.float32)
            routed = ops.moe_route(logits, self.top, self.n_groups, self.group_keep, self.renormalize, self.score)
        chosen, weight = routed
        parts = row_of = None
        on_input = self.weight_on_input
        if self.tensor_cores:
            plan = ops.moe_sort_padded(chosen, self.n_experts, self.tile_rows(x.shape[0]))
            xp = ops.moe_gather(x, plan, weight if on_input else None)
            E, ff, d = self.n_experts, self.intermediate, self.hidden
            if self.gated:
                h = ops.gemm_tcgen05_grouped(xp, self.gate_up.view(E * 2 * ff, d), plan, torch.bfloat16, swiglu=True, status=rt.status)
            else:
                h = ops.gemm_tcgen05_grouped(xp, self.up.view(E * ff, d), plan, torch.bfloat16, status=rt.status, act=self.act)
            if h is not None:
                parts = ops.gemm_tcgen05_grouped(h, self.down.view(E * d, ff), plan, torch.float32, status=rt.status)
                row_of = plan.row_of
        if parts is None:
            plan = ops.moe_sort(chosen, self.n_experts)
            if self.gated:
                h = ops.moe_gemm(0, x, self.gate_up, plan, rt.act_dtype)
            else:
                h = ops.moe_gemm(2, x, self.up, plan, rt.act_dtype, row_scale=weight if on_input else None, act=self.act)
            parts = ops.moe_gemm(1, h, self.down, plan, torch.float32)
            row_of = None
        if accumulate:
            ops.add_(residual, ops.moe_combine(parts, weight, row_of=row_of, unweighted=on_input))
        else:
            ops.moe_combine(parts, weight, out=residual, row_of=row_of, unweighted=on_input)


register_feed_forward("moe", MoEFeedForward)
