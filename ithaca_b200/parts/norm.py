"""RMS norm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, in float32
(src/model.cpp:626-633; GPU kernel src/gpu_kernels.cpp:1177-1195).

Layer norm: y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared
deviations, in float32.  A norm may also stand behind a sublayer: ``add_into`` then adds
``mult * y`` to the residual stream in the same kernel.  The RMS norm may carry a second vector
(``scale``, a per-channel "layer scale") that multiplies what it adds to the stream.  With ``scalar_weight`` the RMS
norm's weight is ONE number for all coordinates (stored as a tensor without dimensions); the kernels get it spread out."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_norm


class RMSNorm:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        out = {spec.weights["weight"]: TensorReq(() if spec.get("scalar_weight") else (spec["size"],), init="ones")}
        if "scale" in spec.weights:
            out[spec.weights["scale"]] = TensorReq((spec["size"],), init="ones")
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = as_float32(tensors[spec.weights["weight"]], runtime)
        if spec.get("scalar_weight"):
            self.weight = self.weight.reshape(1).expand(self.size).contiguous()
        self.scale = as_float32(tensors[spec.weights["scale"]], runtime) if "scale" in spec.weights else None
        self.runtime = runtime

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if x.dim() == 3:                  # several streams per token [T, n, d]: the norm of their plain sum
            return ops.hyper_read(x, None, self.weight, self.eps, out_dtype or self.runtime.act_dtype, rows_in=rows)
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.runtime.act_dtype, rows_in=rows)

    def add_into(self, x: torch.Tensor, residual: torch.Tensor, mult: float = 1.0, copy: Optional[torch.Tensor] = None) -> None:
        """residual += mult * scale * norm(x); ``copy`` receives the new residual in its own type."""
        ops.rmsnorm_add(x, self.weight, self.eps, residual, scale=self.scale, mult=mult, copy=copy)


class LayerNorm:
    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        return {spec.weights["weight"]: TensorReq((spec["size"],), init="ones"),
                spec.weights["bias"]: TensorReq((spec["size"],))}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = as_float32(tensors[spec.weights["weight"]], runtime)
        self.bias = as_float32(tensors[spec.weights["bias"]], runtime)
        self.runtime = runtime

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return ops.layernorm(x, self.weight, self.bias, self.eps, out_dtype or self.runtime.act_dtype, rows_in=rows)

    def add_into(self, x: torch.Tensor, residual: torch.Tensor, mult: float = 1.0) -> None:
        """residual += mult * norm(x)"""
        ops.layernorm(x, self.weight, self.bias, self.eps, torch.float32, into=residual, mult=mult)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
