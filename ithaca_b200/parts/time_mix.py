"""Token-shift time mixing: a recurrent mixer whose matrix state decays per key channel, with a bonus for the current token.

With x' the mixer's input one position earlier in the same sequence (zeros at position 0), each of r, k, v, g, w reads its
own mix m_s = x + (x' - x) * mu_s.  r, k, v = W m (``n_heads`` heads of ``head_dim``), gate = silu(Wg m_g), and one decay
per head and key channel, w = exp(-exp(W2 tanh(W1 m_w) + w0)) with W1 of ``decay_rank`` rows.  Per head, with S of size
head_dim x head_dim and zero before the sequence's first token:

    o = (S + diag(bonus) k v^T)^T r;    S <- diag(w) S + k v^T

so the current token reaches its own read-out through the bonus only.  Every head's o is divided by its root mean square
(``norm_eps`` inside the root); the heads side by side are multiplied by a weight of size heads * head_dim and by the gate,
and projected out.

Per sequence and cache entry the mixer keeps S as float32 [2, heads, head_dim, head_dim] (two copies by the parity of the
position the state belongs to, as the other recurrences do, so that a decode step never overwrites what it read) and the
input of the last position, float32 [2, hidden] by that position's parity.  The mixes, the four wide products (one batched
launch for a few tokens, four launches of the wide-tile product for a prompt), the decay's two small products with tanh between them, the decays, the recurrence and the output norm: everything behind the products is float32 on both paths; only the products'
operands are 16-bit on the bfloat16 path.

The mixer serves alone or as a branch of a composite (``parts/parallel.py``); as a branch it reads the composite's input
itself (``reads_input``), since its products take the shifted mixes, not the input.  It writes its result into a matrix of
its own (a composite that norms every branch before the sum gives it one); a constant on the result, or a column range of
a wider matrix as a plain sum of branches would hand it, is refused.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache.cache import LayerCache, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorReq
from .base import Runtime, as_float32, register_mixer, to_device
from .linear import Linear

STATE, SHIFT = "shift_decay_state", "shift_last_input"
MIXES = ("r", "k", "v", "g", "w")


class ShiftDecayMixer:
    graph_safe = True       # slots, positions and lengths come from device arrays; state and last input by parity
    reads_input = True
    n_in = 0

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorReq]:
        d, H, D, rank = spec["hidden_size"], spec["n_heads"], spec["head_dim"], spec["decay_rank"]
        w = spec.weights
        out = {w[f"mu_{s}"]: TensorReq((d,), std=0.3) for s in MIXES}
        out.update({w[s]: TensorReq((H * D, d)) for s in ("r", "k", "v", "g")})
        out.update({w["w1"]: TensorReq((rank, d)), w["w2"]: TensorReq((H * D, rank)), w["w0"]: TensorReq((H * D,), std=0.5),
                    w["u"]: TensorReq((H, D), std=0.5), w["norm"]: TensorReq((H * D,), init="ones"), w["o"]: TensorReq((d, H * D))})
        return out

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime, standalone: bool = True):
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.head_dim = int(spec["head_dim"])
        self.rank = int(spec["decay_rank"])
        self.norm_eps = float(spec["norm_eps"])
        if self.head_dim > 512:
            raise ValueError(f"shift_decay: the kernel holds a state column's rows in the registers of up to 32 lanes, 16 each; found {self.head_dim}")
        H, D = self.n_heads, self.head_dim
        w = spec.weights
        self.mu = torch.stack([tensors[w[f"mu_{s}"]].to(torch.float32) for s in MIXES]).to(runtime.device).contiguous()     # [5, d]
        wdt = torch.bfloat16 if runtime.dtype == "bfloat16" else torch.float32
        # r, k, v, g as a batch of four products over the four mixes
        self.rkvg = torch.stack([to_device(tensors[w[s]], runtime).to(wdt) for s in ("r", "k", "v", "g")]).contiguous()      # [4, H D, d]
        self.w1 = Linear([tensors[w["w1"]]], runtime)
        self.w2 = Linear([tensors[w["w2"]]], runtime)
        self.w0 = as_float32(tensors[w["w0"]], runtime)
        self.bonus = as_float32(tensors[w["u"]], runtime).reshape(-1).contiguous()
        self.norm_w = as_float32(tensors[w["norm"]], runtime)
        self._out = tensors[w["o"]]
        self.n_mid = H * D
        if standalone:
            self.o = Linear([self._out], runtime)
        self.runtime = runtime

    def cache_requests(self) -> List[object]:
        return [StateRequest(STATE, (2, self.n_heads, self.head_dim, self.head_dim), "float32"),
                StateRequest(SHIFT, (2, self.hidden), "float32")]

    def branch_in(self):
        return []

    def branch_out(self):
        return self._out

    def core(self, p: Optional[torch.Tensor], mid: torch.Tensor, ctx, cache: LayerCache, writes_cache: bool = True, mult: float = 1.0,
             x: Optional[torch.Tensor] = None) -> None:
        """``x`` [T, hidden]: the mixer's input; ``mid`` [T, heads * head_dim] receives the normed, gated heads."""
        if not writes_cache:
            raise ValueError("shift_decay: a run cannot read another run's state without advancing it")
        if mult != 1.0:
            raise ValueError("shift_decay: a constant on the branch's result is not built in")
        rt, H, D = self.runtime, self.n_heads, self.head_dim
        T = x.shape[0]
        mixes = ops.token_shift(x, self.mu, cache.state(SHIFT), ctx)                          # [5, T, d]
        proj = torch.empty((T, 4 * H * D), dtype=torch.float32, device=x.device)             # [r | k | v | g]
        if T > 16:
            # a prompt's portion: each of the four on the product kernel that takes wide token tiles
            from .linear import gemm
            for i in range(4):
                gemm(mixes[i], self.rkvg[i], out=proj[:, i * H * D:(i + 1) * H * D])
        else:
            # a few tokens: the four as one batched launch
            ops.gemm_heads(mixes[:4].permute(1, 0, 2), self.rkvg, proj.view(T, 4, H * D))
        if rt.dtype == "bfloat16":
            from ..csrc import gemm_bf16
            low = gemm_bf16.gemm_act(mixes[4], self.w1.weight, "tanh", rt.act_dtype)          # tanh in the product's epilogue
        else:
            low = ops.plain_act(self.w1(mixes[4], out_dtype=torch.float32), rt.act_dtype, "tanh")
        dec = ops.decay_rows(self.w2(low, out_dtype=torch.float32), self.w0, "double_exp")
        o = ops.row_decay("bonus", proj, 0, H * D, 2 * H * D, dec, None, self.bonus, cache.state(STATE), ctx, H, H, D, D)
        ops.head_norm_gate_into(o, self.norm_w, self.norm_eps, proj, 3 * H * D, H, mid, gate="silu")

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual: torch.Tensor, writes_cache: bool = True,
                accumulate: bool = True) -> None:
        mid = torch.empty((x.shape[0], self.n_mid), dtype=self.runtime.act_dtype, device=x.device)
        self.core(None, mid, ctx, cache, writes_cache, x=x)
        self.o(mid, out=residual, accumulate=accumulate)


register_mixer("shift_decay", ShiftDecayMixer)
