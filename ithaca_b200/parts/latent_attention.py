"""Latent attention: softmax attention whose keys and values are kept as one low-rank latent per token.

q = Wq x, per head [``head_dim`` plain | ``rope_dim`` turning].  Wdkv x has ``kv_rank`` + ``rope_dim`` values: the first
``kv_rank``, RMS-normed with a weight (``norm_eps`` inside the root), are the latent c; the rest is ONE turning key part
that all heads share.  A head's plain key is Wuk c, its value Wuv c.  The turning parts of q and k are rotated by the
position part (all ``rope_dim`` of them); the score is (q_plain . k_plain + q_turn . k_turn) * scale over the keys the
window allows; ordinary softmax; the heads side by side times sigmoid(Wg x) (``head_gate: "wide"``) go through the output
projection.

Only [c | turned key part] is cached, as one key/value head of size kv_rank + rope_dim, and nothing else is ever formed
for a cached token: q_plain is carried into the latent's space (Wuk^T q_plain, one small product per head), attention
runs over the cached rows with the latent as key AND value, and the head's weighted sum of latents is brought to value
space by Wuv (again one small product per head).  Prefill and decode run the same steps.

A layer may read the rows that another layer of equal ``kv_rank``, ``rope_dim`` and rotation has written instead of
making its own (the schedule gives it that layer's cache entry with ``writes_cache=False``): it then has no Wdkv and no
latent norm, but its own Wuk, Wuv, queries, window and everything else (``own_latent: False``).

``rope_dim: 0``: no turning part at all (no position part is needed; the cached row is the latent alone).  ``q_rank``: the
queries come through a latent of their own, q = Wuq (rmsnorm(Wdq x) * w) with Wdq of ``q_rank`` rows (tensors ``dq``,
``dq_norm``, ``uq`` instead of ``q``); it needs ``rope_dim: 0``.
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..cache.cache import KVRequest, LayerCache
from ..config.spec import PartSpec
from ..csrc import attention_latent, ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_mixer, to_device
from .linear import Linear


class LatentAttention:
    graph_safe = True       # reads slots, positions and lengths from device arrays only

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, H, dk, dr, dv, rank = (spec["hidden_size"], spec["n_heads"], spec["head_dim"], spec["rope_dim"], spec["v_head_dim"],
                                  spec["kv_rank"])
        w = spec.weights
        out = {w["uk"]: TensorReq((H * dk, rank)), w["uv"]: TensorReq((H * dv, rank)), w["o"]: TensorReq((d, H * dv))}
        q_rank = spec.get("q_rank")
        if q_rank:
            out.update({w["dq"]: TensorReq((q_rank, d)), w["dq_norm"]: TensorReq((q_rank,), init="ones"),
                        w["uq"]: TensorReq((H * dk, q_rank), std=q_rank ** -0.5)})
        else:
            out[w["q"]] = TensorReq((H * (dk + dr), d))
        if spec.get("own_latent", True):
            out[w["dkv"]] = TensorReq((rank + dr, d))
            out[w["dkv_norm"]] = TensorReq((rank,), init="ones")
        if spec.get("head_gate"):
            out[w["g"]] = TensorReq((H * dv, d))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, position=None):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.head_dim = int(spec["head_dim"])
        self.rope_dim = int(spec["rope_dim"])
        self.v_head_dim = int(spec["v_head_dim"])
        self.rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.norm_eps = float(spec["norm_eps"])
        self.window = spec.get("window")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"latent_attention: window must be positive, found {self.window}")
        self.own_latent = bool(spec.get("own_latent", True))
        gate = spec.get("head_gate")
        if gate not in (None, False, "wide"):
            raise ValueError(f"latent_attention: head_gate {gate!r} is not supported (wide)")
        self.gate = bool(gate)
        self.q_rank = int(spec.get("q_rank") or 0)
        if self.rope_dim == 0:
            position = None
        elif position is None or position.rotary_dim != self.rope_dim or position.pairing != 1 or getattr(position, "magnitude", 1.0) != 1.0:
            raise ValueError("latent_attention: the turning part needs a rotary position part over all of rope_dim with neighbouring pairs")
        if self.q_rank and self.rope_dim:
            raise ValueError("latent_attention: queries through a latent of their own are built for rope_dim 0 only")
        if self.rank > 512:
            raise ValueError(f"latent_attention: the attention kernel keeps up to 512 values of a head's result; kv_rank is {self.rank}")
        self.position = position
        H, dk, dr, dv, rank = self.n_heads, self.head_dim, self.rope_dim, self.v_head_dim, self.rank
        w = spec.weights
        first = tensors[w["dq"]] if self.q_rank else tensors[w["q"]]
        mats = [first] + ([tensors[w["dkv"]]] if self.own_latent else []) + ([tensors[w["g"]]] if self.gate else [])
        self.in_proj = Linear(mats, runtime)
        self.o = Linear([tensors[w["o"]]], runtime)
        if self.q_rank:
            self.uq = Linear([tensors[w["uq"]]], runtime)
            self.q_norm_w = as_float32(tensors[w["dq_norm"]], runtime)
        self.c_off = self.q_rank if self.q_rank else H * (dk + dr)
        self.g_off = self.c_off + (rank + dr if self.own_latent else 0)
        wdt = torch.bfloat16 if runtime.dtype == "bfloat16" else None
        uk = to_device(tensors[w["uk"]], runtime)
        uv = to_device(tensors[w["uv"]], runtime)
        # per head: Wuk^T [rank, dk] multiplies the plain query; Wuv [dv, rank] multiplies the head's sum of latents
        self.uk_t = uk.view(H, dk, rank).transpose(1, 2).contiguous().to(wdt or uk.dtype)
        self.uv = uv.view(H, dv, rank).contiguous().to(wdt or uv.dtype)
        self.c_norm_w = as_float32(tensors[w["dkv_norm"]], runtime) if self.own_latent else None
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        # one key/value head whose rows are [latent | turned key part]; the values are the rows' leading kv_rank columns
        return [KVRequest(1, self.rank + self.rope_dim, self.window, values_in_keys=True)]

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        if writes_cache and not self.own_latent:
            raise ValueError("latent_attention: a layer without a latent of its own cannot write rows")
        rt, H, dk, dr, dv, rank = self.runtime, self.n_heads, self.head_dim, self.rope_dim, self.v_head_dim, self.rank
        T, hd = x.shape[0], rank + dr
        p = self.in_proj(x, out_dtype=torch.float32)                       # [T, q (or its latent) | (c, key part) | g]
        q_full = torch.empty((T, H * hd), dtype=rt.act_dtype, device=x.device)
        table = ctx.tables[cache.kv_group]
        if self.q_rank:
            cq = ops.rmsnorm_range(p[:, :self.q_rank], self.q_norm_w, self.norm_eps, rt.act_dtype)
            q_plain = self.uq(cq, out_dtype=rt.act_dtype)
            if writes_cache:
                ops.latent_append(p, self.c_off, self.c_norm_w, self.norm_eps, cache.k_pages, ctx.token_seq, ctx.token_pos, table,
                                  rank, rt.status)
        else:
            q_plain = torch.empty((T, H * dk), dtype=rt.act_dtype, device=x.device)
            ops.latent_prepare(p, 0, self.c_off, self.c_norm_w, self.norm_eps, q_plain, q_full, cache.k_pages, ctx.token_seq,
                               ctx.token_pos, table, self.position.inv_freq if dr else None, H, dk, dr, rank, writes_cache, rt.status)
        ops.gemm_heads(q_plain.view(T, H, dk), self.uk_t, q_full.view(T, H, hd)[:, :, :rank])
        # [T, H * rank]: the tensor-core kernel whose tile rows are the heads, or (32-bit, other sizes) the CUDA cores
        att = attention_latent.attend(q_full, cache.k_pages, ctx, table, H, self.scale, self.window or 0, rt.status, rank)
        if att is None:
            att = ops.attention_simt(q_full, cache.k_pages, None, ctx.token_seq, ctx.token_pos, table, H, self.scale,
                                     self.window or 0, rt.status, values_in_keys=rank)
        heads = torch.empty((T, H * dv), dtype=rt.act_dtype, device=x.device)
        ops.gemm_heads(att.view(T, H, rank), self.uv, heads.view(T, H, dv))
        if self.gate:
            ops.head_gate(heads, p, self.g_off, heads, H, wide=True)
        self.o(heads, out=residual, accumulate=accumulate)


register_mixer("latent_attention", LatentAttention)
