"""Gated feed-forward: g = Wg x, u = Wu x, h = act(g) * u, y = Wd h, added to the
residual stream (src/model.cpp:1559-1565; silu(x) = x / (1 + exp(-x)), :1309).
Gate and up are stacked into one product ([gate; up], the split the reference
applies to a fused ``ffn_up``, src/model.cpp:1553-1557).

``activation: "swish"`` is the same arrangement with the gate's constants as parameters: g <- min(g, limit) and
u <- clamp(u, -limit, limit) when ``limit`` is given, then h = g * sigmoid(alpha g) * (u + up_shift).

The ungated feed-forward (``mlp``): y = Wd act(Wu x) with ``activation`` ``relu2`` (the square of relu) or ``gelu_tanh``
(0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))), computed in float on the up product's float result."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, register_feed_forward
from .linear import Linear


class GatedMLP:
    graph_safe = True

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, ff = spec["hidden_size"], spec["intermediate_size"]
        w = spec.weights
        return {w["gate"]: TensorReq((ff, d)), w["up"]: TensorReq((ff, d)), w["down"]: TensorReq((d, ff))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        act = spec.get("activation", "silu")
        if act not in ("silu", "swish"):
            raise ValueError(f"gated_mlp: activation {act!r} is not supported (silu, swish)")
        # None: silu(g) * u by the kernels that have always done it; else (alpha, limit or 0, shift)
        self.glu = None if act == "silu" else (float(spec.get("alpha", 1.0)), float(spec.get("limit") or 0.0),
                                               float(spec.get("up_shift", 0.0)))
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        w = spec.weights
        self.gate_up = Linear([tensors[w["gate"]], tensors[w["up"]]], runtime)
        self.down = Linear([tensors[w["down"]]], runtime)
        self.runtime = runtime
        # bfloat16 path: rows interleaved (gate 0, up 0, gate 1, up 1, ...) so that the product's epilogue
        # can apply silu(gate) * up itself and the [tokens, 2 ff] intermediate never exists
        self.fused = runtime.dtype == "bfloat16"
        if self.fused:
            ff, d = self.intermediate, self.hidden
            wgu = self.gate_up.weight
            self.gate_up.weight = torch.stack((wgu[:ff], wgu[ff:]), dim=1).reshape(2 * ff, d).contiguous()

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, accumulate: bool = True) -> None:
        if self.fused:
            from ..csrc import gemm_bf16
            h = gemm_bf16.gemm_swiglu(x, self.gate_up.weight, self.runtime.act_dtype, glu=self.glu)
        else:
            gu = self.gate_up(x, out_dtype=torch.float32)
            h = ops.swiglu(gu, self.runtime.act_dtype) if self.glu is None else ops.glu_act(gu, self.runtime.act_dtype, *self.glu)
        self.down(h, out=residual, accumulate=accumulate)


class PlainMLP:
    graph_safe = True

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, ff = spec["hidden_size"], spec["intermediate_size"]
        w = spec.weights
        return {w["up"]: TensorReq((ff, d)), w["down"]: TensorReq((d, ff))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.act = spec.get("activation", "relu2")
        if self.act not in ops.PLAIN_ACTS:
            raise ValueError(f"mlp: activation {self.act!r} is not supported ({', '.join(ops.PLAIN_ACTS)})")
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        w = spec.weights
        self.up = Linear([tensors[w["up"]]], runtime)
        self.down = Linear([tensors[w["down"]]], runtime)
        self.runtime = runtime

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, accumulate: bool = True) -> None:
        if self.runtime.dtype == "bfloat16":
            from ..csrc import gemm_bf16
            h = gemm_bf16.gemm_act(x, self.up.weight, self.act, self.runtime.act_dtype)     # the activation is the product's epilogue
        else:
            h = ops.plain_act(self.up(x, out_dtype=torch.float32), self.runtime.act_dtype, self.act)
        self.down(h, out=residual, accumulate=accumulate)


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("mlp", PlainMLP)
