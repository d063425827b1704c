"""The gated delta rule mixer.

q = Wq x and k = Wk x (``n_qk_heads`` heads of ``head_dim``), v = Wv x (``n_heads`` heads of ``v_head_dim``); value head h uses
q/k head h / (n_heads / n_qk_heads).  Each of q, k, v passes a short causal convolution over time per channel
(``conv_taps`` taps, no bias; the last column of the stored [channels, taps] matrix meets the current token, zeros stand
before the sequence's start) and silu.  q and k then become unit vectors per head, x / sqrt(sum x^2 + ``unit_eps``), and q
is multiplied by head_dim^(-1/2).  Per token and value head a step b = sigmoid(Wb x) and a decay
g = exp(-exp(A_log) * softplus(Wa x + dt_bias)).  Per head, with S of size head_dim x v_head_dim and zero before the
sequence's first token:

    S <- g S;    u = b (v - S^T k);    S <- S + k u^T;    o = S^T q

so the read-out sees the current token's write.  Every head's o is RMS-normed over its values (``norm_eps`` inside the
root) with one weight of size v_head_dim that the heads share, multiplied by silu(Wg x), and projected out.

Per sequence and cache entry the mixer keeps S as float32 [2, heads, v_head_dim, head_dim], a column's rows side by side
(a column is a recurrence of its own and the kernel gives it to a few lanes; two copies by the parity of
the position the state belongs to, so that a decode step never overwrites what it read and may be run twice) and a ring
of the last ``conv_taps`` inputs of the convolution, float32.  One product gives [q | k | v | g | b | a] in float; the
convolution's result, the unit norms, steps, decays, the state and its sums are float32 on both paths; only the
products' operands are 16-bit on the bfloat16 path.

``decay: "channel"``: one decay per head AND key channel instead of one per head, acting on the rows of S that belong to
the key channels: g = exp(-exp(A_log_h) * softplus(Wa2 (Wa1 x) + dt_bias)) laid out heads x head_dim, with Wa1 of
``decay_rank`` rows (tensors ``a1``, ``a2`` instead of ``a``; ``dt_bias`` of size heads * head_dim).  ``gate``: ``silu`` of a
full projection (``g``), or ``sigmoid_lowrank``: sigmoid(Wg2 (Wg1 x)) with Wg1 of ``gate_rank`` rows (tensors ``g1``, ``g2``).
The small first factors ride in the one input product; the second factors are products of their own on its columns.
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

STATE, RING = "delta_state", "delta_conv_ring"


class GatedDeltaRule:
    graph_safe = True       # slots, positions and lengths come from device arrays; state by parity, ring by position

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, H, G, dk, dv, taps = (spec["hidden_size"], spec["n_heads"], spec["n_qk_heads"], spec["head_dim"], spec["v_head_dim"],
                                 spec["conv_taps"])
        w = spec.weights
        out = {w["q"]: TensorReq((G * dk, d)), w["k"]: TensorReq((G * dk, d)), w["v"]: TensorReq((H * dv, d)),
               w["q_conv"]: TensorReq((G * dk, taps), std=1.0 / taps), w["k_conv"]: TensorReq((G * dk, taps), std=1.0 / taps),
               w["v_conv"]: TensorReq((H * dv, taps), std=1.0 / taps), w["b"]: TensorReq((H, d)),
               w["A_log"]: TensorReq((H,), std=0.5), w["norm"]: TensorReq((dv,), init="ones"), w["o"]: TensorReq((d, H * dv))}
        if spec.get("decay", "head") == "channel":
            r = spec["decay_rank"]
            out.update({w["a1"]: TensorReq((r, d)), w["a2"]: TensorReq((H * dk, r), std=0.2), w["dt_bias"]: TensorReq((H * dk,), std=0.5)})
        else:
            out.update({w["a"]: TensorReq((H, d)), w["dt_bias"]: TensorReq((H,), std=0.5)})
        if spec.get("gate", "silu") == "sigmoid_lowrank":
            r = spec["gate_rank"]
            out.update({w["g1"]: TensorReq((r, d)), w["g2"]: TensorReq((H * dv, r), std=0.2)})
        else:
            out[w["g"]] = TensorReq((H * dv, d))
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.n_qk_heads = int(spec["n_qk_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_head_dim = int(spec["v_head_dim"])
        self.taps = int(spec["conv_taps"])
        self.norm_eps = float(spec["norm_eps"])
        self.unit_eps = float(spec.get("unit_eps", 1e-6))
        if self.n_heads % self.n_qk_heads:
            raise ValueError(f"gated_delta: {self.n_heads} heads cannot share {self.n_qk_heads} query/key heads evenly")
        if self.head_dim > 512:
            raise ValueError(f"gated_delta: the kernel holds a state column's rows in the registers of up to 32 lanes, 16 each; found {self.head_dim}")
        if self.taps < 1:
            raise ValueError("gated_delta: the convolution needs at least one tap")
        H, G, dk, dv = self.n_heads, self.n_qk_heads, self.head_dim, self.v_head_dim
        w = spec.weights
        decay, gate = spec.get("decay", "head"), spec.get("gate", "silu")
        if decay not in ("head", "channel") or gate not in ("silu", "sigmoid_lowrank"):
            raise ValueError(f"gated_delta: decay {decay!r} / gate {gate!r} is not supported (head, channel / silu, sigmoid_lowrank)")
        self.channel_decay, self.lowrank_gate = decay == "channel", gate == "sigmoid_lowrank"
        self.decay_rank = int(spec["decay_rank"]) if self.channel_decay else 1
        self.gate_rank = int(spec["gate_rank"]) if self.lowrank_gate else H * dv
        # one product: [q | k | v | gate (full, or its first factor) | b | decay (per head, or its first factor)]
        roles = ["q", "k", "v", "g1" if self.lowrank_gate else "g", "b", "a1" if self.channel_decay else "a"]
        self.in_proj = Linear([tensors[w[r]] for r in roles], runtime)
        self.a2 = Linear([tensors[w["a2"]]], runtime) if self.channel_decay else None
        self.g2 = Linear([tensors[w["g2"]]], runtime) if self.lowrank_gate else None
        self.o = Linear([tensors[w["o"]]], runtime)
        self.k_off = G * dk
        self.v_off = 2 * G * dk
        self.channels = 2 * G * dk + H * dv
        self.g_off = self.channels
        self.b_off = self.g_off + self.gate_rank
        self.a_off = self.b_off + H
        cw = torch.cat([tensors[w[r]].to(torch.float32) for r in ("q_conv", "k_conv", "v_conv")], dim=0)
        self.conv_w = cw.to(runtime.device).t().contiguous()                  # tap-major [taps, channels]
        self.A_log = as_float32(tensors[w["A_log"]], runtime)
        self.dt_bias = as_float32(tensors[w["dt_bias"]], runtime)
        self.norm_w = as_float32(tensors[w["norm"]], runtime)
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        out: List[object] = [StateRequest(STATE, (2, self.n_heads, self.v_head_dim, self.head_dim), "float32")]
        if self.taps > 1:
            out.append(StateRequest(RING, (self.taps, self.channels), "float32"))
        return out

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        if not writes_cache:
            raise ValueError("gated_delta: a run cannot read another run's state without advancing it")
        rt, H, G, dk, dv = self.runtime, self.n_heads, self.n_qk_heads, self.head_dim, self.v_head_dim
        p = self.in_proj(x, out_dtype=torch.float32)                           # [T, q | k | v | g | b | a]
        ring = cache.state(RING) if self.taps > 1 else None
        u = ops.causal_conv(p[:, :self.channels], self.conv_w, None, ring, ctx, torch.float32, act=True)
        if self.channel_decay:
            bg = ops.delta_prepare(u, 0, self.k_off, p, self.b_off, -1, None, None, G, dk, H, dk ** -0.5, self.unit_eps)
            low = ops.cast(p[:, self.a_off:self.a_off + self.decay_rank], rt.act_dtype)
            dec = ops.decay_rows(self.a2(low, out_dtype=torch.float32), self.dt_bias, "softplus", self.A_log, dk)
            o = ops.row_decay("delta", u, 0, self.k_off, self.v_off, dec, bg[:, 0], None, cache.state(STATE), ctx, H, G, dk, dv)
        else:
            bg = ops.delta_prepare(u, 0, self.k_off, p, self.b_off, self.a_off, self.A_log, self.dt_bias, G, dk, H, dk ** -0.5,
                                   self.unit_eps)
            o = ops.delta_rule(u, 0, self.k_off, self.v_off, bg, cache.state(STATE), ctx, H, G, dk, dv)
        if self.lowrank_gate:
            gate = self.g2(ops.cast(p[:, self.g_off:self.g_off + self.gate_rank], rt.act_dtype), out_dtype=torch.float32)
            mid = ops.head_norm_gate(o, self.norm_w, self.norm_eps, gate, 0, H, rt.act_dtype, gate="sigmoid")
        else:
            mid = ops.head_norm_gate(o, self.norm_w, self.norm_eps, p, self.g_off, H, rt.act_dtype, gate="silu")
        self.o(mid, out=residual, accumulate=accumulate)


register_mixer("gated_delta", GatedDeltaRule)
