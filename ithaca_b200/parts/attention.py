"""Grouped-query attention over the paged cache.

Per token: q, k, v projections; rotary encoding of q and k; k and v appended to the
sequence's pages; attention of each query head over the keys of its kv head
(head h uses kv head h / (n_heads / n_kv_heads)) from position j0 to its own, where
j0 = pos + 1 - window under a window and 0 otherwise; output projection added to
the residual stream.  Scores are (q . k) * scale with scale = 1/sqrt(head_dim)
unless the spec gives one; softmax and the weighted sum are float32
(src/model.cpp:1479-1535; GPU path src/model.cpp:1164-1216).

The three projections are stacked into one product, as the reference does for a
fused ``attn_qkv`` tensor (src/model.cpp:1164-1170).

Options a spec may give (all off by default):

* ``v_head_dim``: value heads of another size than the key heads; the output projection then
  takes n_heads * v_head_dim.
* ``softcap``: scores become cap * tanh(score / cap) after the scale, before the mask.
* ``conv_taps`` with the tensors ``q_conv``, ``k_conv``, ``v_conv`` [channels, taps]: a short causal
  convolution over time on every channel of q, k and v, directly behind the projections and in
  front of the rotation.  The last projected values of a sequence are part of its state: a ring
  of ``taps`` positions per sequence beside its pages (``StateRequest``).
* ``qk_norm: "projection"`` with the tensors ``q_norm``, ``k_norm``: q and k are RMS-normed over their whole
  projections (all heads at once, ``norm_eps`` inside the root) with weights of that size, before the rotation.
  ``qk_norm: "head"``: every head is normed over its own values with one weight of the head's size that all heads share.
* ``head_gate`` with the tensor ``g`` [n_heads, hidden]: every head's result is multiplied by the sigmoid of one
  number per head, a projection of the mixer's input, before the output projection.  ``head_gate: "wide"``: the gate has
  one number per value, ``g`` is [n_heads * v_head_dim, hidden].
* ``sink``: the softmax's denominator counts one more key of score 0 that carries no value: the weights are
  exp(s_j) / (1 + sum exp(s_j)), so a query may attend to nothing.  ``sink: "learned"`` with the tensor ``sink`` [n_heads]:
  every head's sink has a score of its own (not scaled), the denominator's extra term is exp(sink_h).
* ``bias`` with the tensors ``q_bias``, ``k_bias``, ``v_bias``, ``o_bias``: the four projections add a vector.
* ``v_norm``: every value head is divided by its root mean square (``norm_eps`` inside the root, no weight) and cached so.
* a position part whose cos and sin carry a constant factor (``magnitude``).

With any of these but the first three the mixer runs "wide": one product gives [q | k | v | g] in float, one kernel norms, rotates
and appends, the attention kernel runs, and the gate kernel writes the output projection's operand.  A wide mixer can
also serve as a branch of a composite (``parts/parallel.py``): ``branch_in()`` / ``branch_out()`` hand out its matrices
so that the composite stacks them with other branches' into one product each, and ``core`` works on column ranges of
those products' matrices.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

from ..cache.cache import KVRequest, LayerCache, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_mixer
from .linear import Linear


class Attention:
    graph_safe = True       # reads slots, positions and lengths from device arrays only

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, nh, nkv, hd = spec["hidden_size"], spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        w = spec.weights
        hdv = spec.get("v_head_dim") or hd
        out = {w["q"]: TensorReq((nh * hd, d)), w["k"]: TensorReq((nkv * hd, d)),
               w["v"]: TensorReq((nkv * hdv, d)), w["o"]: TensorReq((d, nh * hdv))}
        if spec.get("qk_norm"):
            per_head = spec.get("qk_norm") == "head"
            out[w["q_norm"]] = TensorReq((hd if per_head else nh * hd,), init="ones")
            out[w["k_norm"]] = TensorReq((hd if per_head else nkv * hd,), init="ones")
        if spec.get("head_gate"):
            out[w["g"]] = TensorReq((nh * hdv if spec.get("head_gate") == "wide" else nh, d))
        if spec.get("sink") == "learned":
            out[w["sink"]] = TensorReq((nh,), std=1.0)
        if spec.get("bias"):
            out[w["q_bias"]], out[w["k_bias"]] = TensorReq((nh * hd,)), TensorReq((nkv * hd,))
            out[w["v_bias"]], out[w["o_bias"]] = TensorReq((nkv * hdv,)), TensorReq((d,))
        taps = spec.get("conv_taps") or 0
        if taps:
            # taps around 1/taps: the convolution keeps the projections' scale
            for role, rows in (("q_conv", nh * hd), ("k_conv", nkv * hd), ("v_conv", nkv * hdv)):
                out[w[role]] = TensorReq((rows, taps), std=1.0 / taps)
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, position=None,
                 standalone: bool = True):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_head_dim = int(spec.get("v_head_dim") or self.head_dim)
        self.softcap = float(spec.get("softcap") or 0.0)
        self.conv_taps = int(spec.get("conv_taps") or 0)
        if self.softcap < 0 or self.conv_taps < 0:
            raise ValueError("attention: softcap and conv_taps cannot be negative")
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads cannot share {self.n_kv_heads} kv heads evenly")
        self.window = spec.get("window")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"attention: window must be positive, found {self.window}")
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = position
        if position is not None and position.rotary_dim > self.head_dim:
            raise ValueError("attention: the rotated width exceeds the head size")
        w = spec.weights
        wq, wk = tensors[w["q"]], tensors[w["k"]]
        qk_norm = spec.get("qk_norm")
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"attention: qk_norm {qk_norm!r} is not supported (projection, head)")
        self.norm_per_head = qk_norm == "head"
        self.head_gate = bool(spec.get("head_gate"))
        self.gate_wide = spec.get("head_gate") == "wide"
        self.sink = bool(spec.get("sink"))
        if spec.get("sink") not in (None, False, True, "learned"):
            raise ValueError(f"attention: sink {spec.get('sink')!r} is not supported (true, learned)")
        # what the kernels get: False, True (a key of score 0) or every head's score
        self.sink_arg = as_float32(tensors[w["sink"]], runtime) if spec.get("sink") == "learned" else self.sink
        self.v_norm = bool(spec.get("v_norm"))
        self.biased = bool(spec.get("bias"))
        self.wide = bool(qk_norm or self.head_gate or self.sink or self.v_norm or self.biased or (position is not None and getattr(position, "magnitude", 1.0) != 1.0)
                         or not standalone)
        if self.wide and self.conv_taps:
            raise ValueError("attention: a short convolution and the wide arrangement (qk_norm, head_gate) do not go together")
        self.norm_eps = float(spec.get("norm_eps") or 0.0)
        self.q_norm_w = as_float32(tensors[w["q_norm"]], runtime) if qk_norm else None
        self.k_norm_w = as_float32(tensors[w["k_norm"]], runtime) if qk_norm else None
        # bfloat16 path with the whole head rotated: the rows of the q and k weights are reordered so that the
        # two members of a rotary pair are neighbours, (i, i + hd/2) -> (2i, 2i + 1).  Scores do not change (q and k
        # are reordered alike, and the cache holds k in that order); the product's epilogue can then rotate a pair
        # and write q and the cache entries itself, without the [tokens, q+k+v] intermediate.
        self.pairing = position.pairing if position is not None else 0
        self.fused_rope = (runtime.dtype == "bfloat16" and position is not None and position.rotary_dim == self.head_dim
                           and self.head_dim % 2 == 0 and not self.conv_taps and self.v_head_dim == self.head_dim
                           and not self.wide)
        if self.fused_rope and self.pairing == 0:
            half = self.head_dim // 2
            order = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)
            wq = wq.view(self.n_heads, self.head_dim, -1)[:, order].reshape(wq.shape)
            wk = wk.view(self.n_kv_heads, self.head_dim, -1)[:, order].reshape(wk.shape)
            self.pairing = 1                                       # pairs are (2i, 2i + 1) from here on
        self._in = [wq, wk, tensors[w["v"]]] + ([tensors[w["g"]]] if self.head_gate else [])
        self._out = tensors[w["o"]]
        self.k_off = self.n_heads * self.head_dim
        self.v_off = self.k_off + self.n_kv_heads * self.head_dim
        self.g_off = self.v_off + self.n_kv_heads * self.v_head_dim
        self.n_mid = self.n_heads * self.v_head_dim
        self.n_in = self.g_off + ((self.n_mid if self.gate_wide else self.n_heads) if self.head_gate else 0)
        # the projections' biases as one vector over the columns of the wide product (the gate has none)
        self.in_bias = None
        self._out_bias = None
        if self.biased:
            zeros = torch.zeros(self.n_in - self.g_off, dtype=torch.float32)
            self.in_bias = torch.cat([tensors[w[r]].to(torch.float32).cpu() for r in ("q_bias", "k_bias", "v_bias")] + [zeros]).to(runtime.device).contiguous()
            self._out_bias = as_float32(tensors[w["o_bias"]], runtime)
        if standalone:
            self.qkv = Linear(self._in, runtime)
            self.o = Linear([self._out], runtime)
        self.runtime = runtime
        self.conv_weight = None
        self.channels = (self.n_heads + self.n_kv_heads) * self.head_dim + self.n_kv_heads * self.v_head_dim
        if self.conv_taps:
            cw = torch.cat([tensors[w[r]].to(torch.float32) for r in ("q_conv", "k_conv", "v_conv")], dim=0)
            self.conv_weight = cw.to(runtime.device).t().contiguous()              # tap-major [taps, channels]: a tap's weights of neighbouring channels lie together
        # the plain path (projections, then convolution, rotation and append in one kernel) serves every option
        self.plain_append = (bool(self.conv_taps) or self.v_head_dim != self.head_dim) and not self.wide

    # -- as a branch of a composite mixer ------------------------------------------------------
    def branch_in(self):
        """The matrices whose products with the mixer's input ``core`` reads, in the order of its columns."""
        return list(self._in)

    def branch_out(self):
        """The matrix that multiplies what ``core`` writes."""
        return self._out

    def branch_out_bias(self):
        """The vector the output projection adds (float32), or None."""
        return self._out_bias

    def core(self, p: torch.Tensor, mid: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True, mult: float = 1.0) -> None:
        """``p`` [T, n_in] float: [q | k | v | g] (a column range of a wider matrix may be given); ``mid`` [T, n_mid] in the
        activation type receives ``mult`` times the gated heads, the operand of the output projection."""
        rt, pos = self.runtime, self.position
        q = torch.empty((p.shape[0], self.n_heads * self.head_dim), dtype=rt.act_dtype, device=p.device)
        table = ctx.tables[cache.kv_group]
        ops.norm_rope_append(p, 0, self.k_off, self.v_off, self.q_norm_w, self.k_norm_w, self.norm_eps, q, cache.k_pages,
                             cache.v_pages, ctx.token_seq, ctx.token_pos, table, pos.inv_freq if pos is not None else None,
                             getattr(pos, "magnitude", 1.0), self.n_heads, pos.rotary_dim if pos is not None else 0,
                             self.pairing, writes_cache, rt.status, per_head=self.norm_per_head, bias=self.in_bias, v_norm=self.v_norm)
        att = attend(q, cache, ctx, table, self.n_heads, self.scale, self.window or 0, rt, self.softcap, sink=self.sink_arg)
        ops.head_gate(att, p if self.head_gate else None, self.g_off, mid, self.n_heads, mult, wide=self.gate_wide)

    def cache_requests(self) -> List[object]:
        v = self.v_head_dim if self.v_head_dim != self.head_dim else None
        out: List[object] = [KVRequest(self.n_kv_heads, self.head_dim, self.window, v)]
        if self.conv_taps > 1:
            out.append(StateRequest("conv_ring", (self.conv_taps, self.channels), "float32"))
        return out

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor,
                writes_cache: bool = True, accumulate: bool = True) -> None:
        """``accumulate=False``: the output replaces what ``residual`` holds instead of adding to it."""
        rt = self.runtime
        T = x.shape[0]
        if self.wide:
            p = self.qkv(x, out_dtype=torch.float32)
            mid = torch.empty((T, self.n_mid), dtype=rt.act_dtype, device=x.device)
            self.core(p, mid, ctx, cache, writes_cache)
            self.o(mid, out=residual, accumulate=accumulate)
            if self._out_bias is not None:
                ops.add_rows_(residual, self._out_bias)
            return
        q = torch.empty((T, self.n_heads * self.head_dim), dtype=rt.act_dtype, device=x.device)
        table = ctx.tables[cache.kv_group]
        pos = self.position
        done = False
        if self.fused_rope:
            key = pos.key
            cos_sin = ctx.shared.get(key)
            if cos_sin is None:                                   # once per step, shared by the layers
                cos_sin = ctx.shared[key] = ops.rope_table(ctx.token_pos, pos.inv_freq)
            done = ops.gemm_qkv_rope(x, self.qkv.weight, q, cache.k_pages, cache.v_pages, cos_sin, ctx.token_seq,
                                     ctx.token_pos, table, self.n_heads, self.n_kv_heads, self.head_dim, writes_cache,
                                     rt.status)
        if self.plain_append:
            qkv = self.qkv(x, out_dtype=torch.float32)
            ring = cache.state("conv_ring") if self.conv_taps > 1 else None
            ops.conv_rope_append(qkv, self.conv_weight, ring, ctx.slots, ctx.cu_seqlens, ctx.kv_lens, q, cache.k_pages,
                                 cache.v_pages, ctx.token_seq, ctx.token_pos, table,
                                 pos.inv_freq if pos is not None else None, self.n_heads, self.n_kv_heads,
                                 pos.rotary_dim if pos is not None else 0, self.pairing, writes_cache, rt.status)
        elif not done:
            qkv = self.qkv(x, out_dtype=torch.float32)
            ops.rope_append(qkv, q, cache.k_pages, cache.v_pages, ctx.token_seq, ctx.token_pos, table,
                            pos.inv_freq if pos is not None else None, self.n_heads, self.n_kv_heads, self.head_dim,
                            pos.rotary_dim if pos is not None else 0, self.pairing, writes_cache, rt.status)
        att = attend(q, cache, ctx, table, self.n_heads, self.scale, self.window or 0, rt, self.softcap)
        self.o(att, out=residual, accumulate=accumulate)


def attend(q: torch.Tensor, cache: LayerCache, ctx, table: torch.Tensor, n_heads: int, scale: float, window: int,
           rt: Runtime, softcap: float = 0.0, sink=False) -> torch.Tensor:
    """Chooses the attention kernel: tensor-core kernels for bfloat16 when they take the
    head sizes, else the CUDA-core kernel (always for float32)."""
    if q.dtype == torch.bfloat16 and cache.v_pages.shape[3] == cache.k_pages.shape[3]:
        from ..csrc import attention_bf16
        out = attention_bf16.attend(q, cache.k_pages, cache.v_pages, ctx, table, n_heads, scale, window, rt.status,
                                    softcap=softcap, sink=sink)
        if out is not None:
            return out
    return ops.attention_simt(q, cache.k_pages, cache.v_pages, ctx.token_seq, ctx.token_pos, table, n_heads, scale,
                              window, rt.status, softcap=softcap, sink=sink)


register_mixer("attention", Attention)
