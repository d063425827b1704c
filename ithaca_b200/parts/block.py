"""The arrangement of a layer's parts around the residual stream.

``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)) -- the order of the
reference's layer loop (src/model.cpp:1460-1565).  The residual stream is float32
and the parts add into it, so the sum never passes through 16 bits.  With ``layer_scale`` in the record's
parameters (``{"mixer": tensor name, "feed_forward": tensor name}``) each sublayer's result is multiplied element by element by
a vector of the layer before it joins the stream: x += s1 * mixer(norm(x)); x += s2 * feed_forward(norm(x)).  The sublayer
then writes into a float32 buffer of its own, and one kernel adds s1 times it to the stream and forms the feed-forward's
norm of the new stream in the same pass.  Such a layer may have no feed-forward.

``sandwich``: a norm in front of and behind each sublayer, and a constant on what joins the
stream: x += m * norm_out(mixer(norm(x))); x += m * norm_out'(feed_forward(norm'(x))).  The
sublayer writes into a float32 buffer of its own (the stream is not what it adds to); the norm
behind it scales and adds in one kernel.  The feed-forward may be absent.

``outnorm``: a norm behind each sublayer only: x += norm_out(mixer(x)); x += norm_out'(feed_forward(x)).  The
sublayers read the stream itself.  On the 16-bit path their operand is a 16-bit copy of the stream, which the
norm's kernel writes beside the float stream it adds to (the next sublayer's input, also across layers), so no
kernel exists only to convert.  The feed-forward may be absent.

``hyper``: n residual streams per token instead of one (the stream tensor is [T, n, d]).  A sublayer f with the layer's
vectors a, b (size n) and matrix M (n x n, indexed [from, to]) reads u = sum_s a_s x_s through its norm and writes all
streams at once from the old ones: x_t <- sum_s M[s, t] x_s + b_t f(norm(u)).  The record's parameters name the tensors:
``{"streams": n, "mixer": {"in": ..., "out": ..., "mix": ...}, "feed_forward": {...}}``.  One kernel reads, one writes;
the write of the mixer's result already forms the feed-forward's operand from the new streams.  The feed-forward may be absent.
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping

import torch

from ..cache.cache import LayerCache
from ..config.spec import BlockSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Runtime, as_float32, register_block


def _merge(into: Dict[str, TensorReq], more: Mapping[str, TensorReq]) -> None:
    for name, req in more.items():
        if name in into and tuple(into[name].shape) != tuple(req.shape):
            raise ValueError(f"tensor '{name}' is asked for with shapes {into[name].shape} and {req.shape}")
        into[name] = req


class PreNormBlock:
    @classmethod
    def manifest(cls, spec: BlockSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        _merge(out, MIXERS.get(spec.mixer.kind).manifest(spec.mixer))
        if spec.feed_forward is not None:
            _merge(out, FEED_FORWARDS.get(spec.feed_forward.kind).manifest(spec.feed_forward))
        for name, n in spec.norms.items():
            if spec.feed_forward is None and name == "feed_forward":
                continue
            _merge(out, NORMS.get(n.kind).manifest(n))
        if spec.position is not None:
            _merge(out, POSITIONS.get(spec.position.kind).manifest(spec.position))
        size = spec.norms["mixer"].get("size")
        for sub, name in (spec.params.get("layer_scale") or {}).items():
            if sub == "mixer" or spec.feed_forward is not None:
                _merge(out, {name: TensorReq((size,), init="ones")})
        return out

    def __init__(self, spec: BlockSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        scales = spec.params.get("layer_scale")
        has_ff = spec.feed_forward is not None
        if not has_ff and scales is None:
            raise ValueError("prenorm block: a layer without layer scale needs a feed-forward")
        for need in ("mixer",) + (("feed_forward",) if has_ff else ()):
            if need not in spec.norms:
                raise ValueError(f"prenorm block: the spec has no '{need}' norm")
        position = None
        if spec.position is not None:
            position = POSITIONS.get(spec.position.kind)(spec.position, tensors, runtime)
        mixer_cls = MIXERS.get(spec.mixer.kind)
        if "position" in inspect.signature(mixer_cls.__init__).parameters:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime, position=position)
        else:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, tensors, runtime) if has_ff else None
        self.mixer_norm = NORMS.get(spec.norms["mixer"].kind)(spec.norms["mixer"], tensors, runtime)
        self.ff_norm = NORMS.get(spec.norms["feed_forward"].kind)(spec.norms["feed_forward"], tensors, runtime) if has_ff else None
        self.runtime = runtime
        self.scaled = scales is not None
        if self.scaled:
            for sub in ("mixer",) + (("feed_forward",) if has_ff else ()):
                if sub not in scales:
                    raise ValueError(f"prenorm block: layer_scale names no vector for the {sub}")
            if has_ff and not (hasattr(self.ff_norm, "weight") and hasattr(self.ff_norm, "eps") and not hasattr(self.ff_norm, "bias")):
                raise ValueError("prenorm block: with layer scale the feed-forward's norm must be an RMS norm")
            self.mixer_scale = as_float32(tensors[scales["mixer"]], runtime)
            self.ff_scale = as_float32(tensors[scales["feed_forward"]], runtime) if has_ff else None

    def cache_requests(self) -> List[object]:
        return list(self.mixer.cache_requests())

    def forward(self, residual: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True) -> None:
        if not self.scaled:
            self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache, residual, writes_cache)
            self.feed_forward.forward(self.ff_norm.forward(residual), ctx, residual)
            return
        y = torch.empty_like(residual)
        self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache, y, writes_cache, accumulate=False)
        if self.feed_forward is None:
            ops.scale_add_norm(y, self.mixer_scale, residual)
            return
        xn = ops.scale_add_norm(y, self.mixer_scale, residual, self.ff_norm.weight, self.ff_norm.eps, self.runtime.act_dtype)
        self.feed_forward.forward(xn, ctx, y, accumulate=False)
        ops.scale_add_norm(y, self.ff_scale, residual)


class SandwichBlock:
    NORMS = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")

    @classmethod
    def manifest(cls, spec: BlockSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        _merge(out, MIXERS.get(spec.mixer.kind).manifest(spec.mixer))
        if spec.feed_forward is not None:
            _merge(out, FEED_FORWARDS.get(spec.feed_forward.kind).manifest(spec.feed_forward))
        for name, n in spec.norms.items():
            if spec.feed_forward is None and name.startswith("feed_forward"):
                continue
            _merge(out, NORMS.get(n.kind).manifest(n))
        if spec.position is not None:
            _merge(out, POSITIONS.get(spec.position.kind).manifest(spec.position))
        return out

    def __init__(self, spec: BlockSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        has_ff = spec.feed_forward is not None
        for need in self.NORMS[:2] + (self.NORMS[2:] if has_ff else ()):
            if need not in spec.norms:
                raise ValueError(f"sandwich block: the spec has no '{need}' norm")
        self.mult = float(spec.params.get("residual_mult", 1.0))
        position = None
        if spec.position is not None:
            position = POSITIONS.get(spec.position.kind)(spec.position, tensors, runtime)
        mixer_cls = MIXERS.get(spec.mixer.kind)
        if "position" in inspect.signature(mixer_cls.__init__).parameters:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime, position=position)
        else:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, tensors, runtime) if has_ff else None

        def norm(name):
            n = spec.norms[name]
            made = NORMS.get(n.kind)(n, tensors, runtime)
            if name.endswith("_out") and not hasattr(made, "add_into"):
                raise ValueError(f"sandwich block: norm kind '{n.kind}' cannot stand behind a sublayer")
            return made

        self.mixer_norm, self.mixer_out_norm = norm("mixer"), norm("mixer_out")
        self.ff_norm, self.ff_out_norm = (norm("feed_forward"), norm("feed_forward_out")) if has_ff else (None, None)

    def cache_requests(self) -> List[object]:
        return list(self.mixer.cache_requests())

    def forward(self, residual: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True) -> None:
        y = torch.empty_like(residual)
        self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache, y, writes_cache, accumulate=False)
        self.mixer_out_norm.add_into(y, residual, self.mult)
        if self.feed_forward is not None:
            self.feed_forward.forward(self.ff_norm.forward(residual), ctx, y, accumulate=False)
            self.ff_out_norm.add_into(y, residual, self.mult)


class OutNormBlock:
    COPY = "stream_copy"        # in StepContext.shared: the stream in the activation type, as of the last add

    @classmethod
    def manifest(cls, spec: BlockSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        _merge(out, MIXERS.get(spec.mixer.kind).manifest(spec.mixer))
        if spec.feed_forward is not None:
            _merge(out, FEED_FORWARDS.get(spec.feed_forward.kind).manifest(spec.feed_forward))
        for name, n in spec.norms.items():
            if spec.feed_forward is None and name.startswith("feed_forward"):
                continue
            _merge(out, NORMS.get(n.kind).manifest(n))
        if spec.position is not None:
            _merge(out, POSITIONS.get(spec.position.kind).manifest(spec.position))
        return out

    def __init__(self, spec: BlockSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        has_ff = spec.feed_forward is not None
        for need in ("mixer_out",) + (("feed_forward_out",) if has_ff else ()):
            if need not in spec.norms:
                raise ValueError(f"outnorm block: the spec has no '{need}' norm")
        self.runtime = runtime
        position = None
        if spec.position is not None:
            position = POSITIONS.get(spec.position.kind)(spec.position, tensors, runtime)
        mixer_cls = MIXERS.get(spec.mixer.kind)
        if "position" in inspect.signature(mixer_cls.__init__).parameters:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime, position=position)
        else:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, tensors, runtime) if has_ff else None

        def norm(name):
            n = spec.norms[name]
            made = NORMS.get(n.kind)(n, tensors, runtime)
            if "copy" not in inspect.signature(getattr(made, "add_into", lambda: None)).parameters:
                raise ValueError(f"outnorm block: norm kind '{n.kind}' cannot stand behind a sublayer and hand the stream on")
            return made

        self.mixer_out_norm = norm("mixer_out")
        self.ff_out_norm = norm("feed_forward_out") if has_ff else None

    def cache_requests(self) -> List[object]:
        return list(self.mixer.cache_requests())

    def _operand(self, residual: torch.Tensor, ctx) -> torch.Tensor:
        """What a sublayer multiplies: the stream itself in float32, its 16-bit copy otherwise."""
        if self.runtime.act_dtype == torch.float32:
            return residual
        x = ctx.shared.pop(self.COPY, None)
        return x if x is not None else ops.cast(residual, self.runtime.act_dtype)

    def _fresh_copy(self, residual: torch.Tensor):
        return None if self.runtime.act_dtype == torch.float32 else torch.empty_like(residual, dtype=self.runtime.act_dtype)

    def forward(self, residual: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True) -> None:
        y = torch.empty_like(residual)
        self.mixer.forward(self._operand(residual, ctx), ctx, cache, y, writes_cache, accumulate=False)
        copy = self._fresh_copy(residual)
        self.mixer_out_norm.add_into(y, residual, copy=copy)
        if copy is not None:
            ctx.shared[self.COPY] = copy
        if self.feed_forward is not None:
            self.feed_forward.forward(self._operand(residual, ctx), ctx, y, accumulate=False)
            copy = self._fresh_copy(residual)
            self.ff_out_norm.add_into(y, residual, copy=copy)
            if copy is not None:
                ctx.shared[self.COPY] = copy


class HyperBlock:
    ROLES = ("in", "out", "mix")

    @classmethod
    def manifest(cls, spec: BlockSpec) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        _merge(out, MIXERS.get(spec.mixer.kind).manifest(spec.mixer))
        if spec.feed_forward is not None:
            _merge(out, FEED_FORWARDS.get(spec.feed_forward.kind).manifest(spec.feed_forward))
        for name, n in spec.norms.items():
            if spec.feed_forward is None and name == "feed_forward":
                continue
            _merge(out, NORMS.get(n.kind).manifest(n))
        if spec.position is not None:
            _merge(out, POSITIONS.get(spec.position.kind).manifest(spec.position))
        n = int(spec.params["streams"])
        for sub in ("mixer",) + (("feed_forward",) if spec.feed_forward is not None else ()):
            names = spec.params[sub]
            # random weights: every stream read and written with about equal weight, the streams mostly kept apart
            _merge(out, {names["in"]: TensorReq((n,), init="ones", std=0.0), names["out"]: TensorReq((n,), init="ones"),
                         names["mix"]: TensorReq((n, n), std=0.5)})
        return out

    def __init__(self, spec: BlockSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        has_ff = spec.feed_forward is not None
        self.n = int(spec.params["streams"])
        if not 1 <= self.n <= 16:
            raise ValueError(f"hyper block: 1 to 16 streams are supported, found {self.n}")
        for need in ("mixer",) + (("feed_forward",) if has_ff else ()):
            if need not in spec.norms or need not in spec.params:
                raise ValueError(f"hyper block: the spec has no '{need}' norm or stream tensors")
        position = None
        if spec.position is not None:
            position = POSITIONS.get(spec.position.kind)(spec.position, tensors, runtime)
        mixer_cls = MIXERS.get(spec.mixer.kind)
        if "position" in inspect.signature(mixer_cls.__init__).parameters:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime, position=position)
        else:
            self.mixer = mixer_cls(spec.mixer, tensors, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, tensors, runtime) if has_ff else None
        self.mixer_norm = NORMS.get(spec.norms["mixer"].kind)(spec.norms["mixer"], tensors, runtime)
        self.ff_norm = NORMS.get(spec.norms["feed_forward"].kind)(spec.norms["feed_forward"], tensors, runtime) if has_ff else None
        for nm in (self.mixer_norm,) + ((self.ff_norm,) if has_ff else ()):
            if not (hasattr(nm, "weight") and hasattr(nm, "eps") and not hasattr(nm, "bias")):
                raise ValueError("hyper block: the norms in front of the sublayers must be RMS norms")
        self.runtime = runtime

        def stream_tensors(sub):
            names = spec.params[sub]
            a, b, m = (as_float32(tensors[names[r]], runtime) for r in self.ROLES)
            if a.numel() != self.n or b.numel() != self.n or tuple(m.shape) != (self.n, self.n):
                raise ValueError(f"hyper block: the {sub}'s stream tensors do not fit {self.n} streams")
            return a, b, m

        self.mixer_in, self.mixer_out, self.mixer_mix = stream_tensors("mixer")
        if has_ff:
            self.ff_in, self.ff_out, self.ff_mix = stream_tensors("feed_forward")

    def cache_requests(self) -> List[object]:
        return list(self.mixer.cache_requests())

    def forward(self, streams: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True) -> None:
        rt = self.runtime
        T, n, d = streams.shape
        xn = ops.hyper_read(streams, self.mixer_in, self.mixer_norm.weight, self.mixer_norm.eps, rt.act_dtype)
        y = torch.empty((T, d), dtype=torch.float32, device=streams.device)
        self.mixer.forward(xn, ctx, cache, y, writes_cache, accumulate=False)
        if self.feed_forward is None:
            ops.hyper_write(streams, y, self.mixer_mix, self.mixer_out)
            return
        xn = ops.hyper_write(streams, y, self.mixer_mix, self.mixer_out, self.ff_in, self.ff_norm.weight, self.ff_norm.eps, rt.act_dtype)
        self.feed_forward.forward(xn, ctx, y, accumulate=False)
        ops.hyper_write(streams, y, self.ff_mix, self.ff_out)


register_block("prenorm", PreNormBlock)
register_block("hyper", HyperBlock)
register_block("sandwich", SandwichBlock)
register_block("outnorm", OutNormBlock)
