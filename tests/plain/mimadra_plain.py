"""A plain, slow Mimadra decoder: whole sequences, no cache, one function per mechanism.

Nothing here is shared with the library under test.  It reads ``config.json`` keys from a plain dictionary and
tensors from a plain name -> tensor mapping and computes on the CPU in the dtype it is given (float64 by default,
so that it is the more exact side of a comparison).

The design in this file's notation (T tokens at positions 0 .. T-1, width d, N the RMS norm with a weight):

* x = E[ids].
* a layer: x += s1 * mixer(N1(x)); x += s2 * ff(N2(x)) with s1, s2 vectors of the layer; a layer may have no ff.
* mixer ``attention``: H query heads over G key/value heads; q and k are RMS-normed per head with one weight of the
  head's size; the leading r dimensions of every q and k head turn in pairs (i, i + r/2) by p * base^(-2i/r);
  scores (q . k) * c over the last w positions (the own one included); weights exp(s_j) / (1 + sum_j exp(s_j));
  the heads side by side times sigmoid(Wg h); output projection.
* mixer ``delta``: q, k (G heads of size dk) and v (H heads of size dv) pass a causal convolution over time per
  channel and silu; q and k are made unit vectors per head (1e-6 inside the root) and q is divided by sqrt(dk);
  b = sigmoid(Wb h), a = exp(-exp(A_log) * softplus(Wa h + dt_bias)), one each per head; per head
  S <- a S; u = b (v - S^T k); S <- S + k u^T; o = S^T q; o is RMS-normed over dv with a weight of that size and
  multiplied by silu(Wg h); output projection.
* mixer ``latent_attention``: q = Wq h, per head [dk plain | dr turning]; Wdkv h = [kv_rank | dr]: the first part
  RMS-normed with a weight is the latent c, the second is one turning key part for all heads; a head's plain key is
  Wuk c, its value Wuv c; the turning parts turn in pairs (2i, 2i + 1) by p * base^(-2i/dr); scores
  (q_plain . k_plain + q_turn . k_turn) * c over the last w positions; ordinary softmax; times sigmoid(Wg h); output
  projection.  A layer with ``kv_from: j`` has no Wdkv and takes c and the turned key part from layer j.
* ff: Wdown relu(Wup h)^2.
* logits = cap * tanh(W N(x) / cap).
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(x.dtype)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def _angles(positions: Sequence[int], r: int, base: float, dtype) -> torch.Tensor:
    # the design forms positions and angles in 32-bit: the frequency is rounded to float32 and so is the product
    p = torch.tensor(list(positions), dtype=torch.float32)[:, None]
    f = torch.tensor([float(base) ** (-2.0 * i / r) for i in range(r // 2)], dtype=torch.float64).to(torch.float32)[None, :]
    return (p * f).to(dtype)                                       # [T, r/2]


def rotate_halves(x: torch.Tensor, positions: Sequence[int], r: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: the pair (i, i + r/2) of every head's leading r dimensions turns by p * base^(-2i/r)."""
    y = x.clone()
    a = _angles(positions, r, base, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :r // 2], x[..., r // 2:r]
    y[..., :r // 2] = u * c - v * s
    y[..., r // 2:r] = v * c + u * s
    return y


def rotate_neighbours(x: torch.Tensor, positions: Sequence[int], r: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: the pair (2i, 2i + 1) of every head's leading r dimensions turns by p * base^(-2i/r)."""
    y = x.clone()
    a = _angles(positions, r, base, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    y[..., 0:r:2] = u * c - v * s
    y[..., 1:r:2] = v * c + u * s
    return y


def windowed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
                       sink: bool) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv].  Query i sees keys j with 0 <= i - j < window.  With
    ``sink`` the weights are exp(s_j) / (1 + sum exp(s_j)): a key of score 0 that carries nothing."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - m)
            den = e.sum() + (math.exp(-m) if sink else 0.0)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + ".q"].T).view(T, H, dk)
    k = (h @ t[p + ".k"].T).view(T, G, dk)
    v = (h @ t[p + ".v"].T).view(T, G, dv)
    q, k = rms_norm(q, t[p + ".q.norm"], eps), rms_norm(k, t[p + ".k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_halves(q, range(T), rot["dims"], rot["base"])
        k = rotate_halves(k, range(T), rot["dims"], rot["base"])
    window = m["mask"]["size"] if m.get("mask") else None
    o = windowed_attention(q, k, v, m["scale"], window, sink=True).reshape(T, H * dv)
    return (o * sigmoid(h @ t[p + ".g"].T)) @ t[p + ".o"].T


def short_convolution(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]: y[p, c] = sum_j w[c, j] x[p - (taps - 1 - j), c], zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * w[:, j]
    return y


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """q, k [T, H, dk] (already per value head), v [T, H, dv], beta, a [T, H] -> [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for h in range(H):
        S = torch.zeros((dk, dv), dtype=q.dtype)
        for i in range(T):
            S = a[i, h] * S
            u = beta[i, h] * (v[i, h] - S.T @ k[i, h])
            S = S + torch.outer(k[i, h], u)
            out[i, h] = S.T @ q[i, h]
    return out


def delta_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ t[p + ".q"].T, t[p + ".q.conv"])).view(T, G, dk)
    k = silu(short_convolution(h @ t[p + ".k"].T, t[p + ".k.conv"])).view(T, G, dk)
    v = silu(short_convolution(h @ t[p + ".v"].T, t[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = sigmoid(h @ t[p + ".b"].T)
    a = torch.exp(-torch.exp(t[p + ".A_log"]) * softplus(h @ t[p + ".a"].T + t[p + ".dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, a)
    o = rms_norm(o, t[p + ".norm"], eps).reshape(T, H * dv) * silu(h @ t[p + ".g"].T)
    return o @ t[p + ".o"].T


def latent_attention_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float,
                           kept: Dict[int, tuple], layer: int) -> torch.Tensor:
    """``kept``: layer -> (latent [T, kv_rank], turned key part [T, dr]) of the layers that made their own."""
    T = h.shape[0]
    H, dk, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ t[p + ".q"].T).view(T, H, dk + dr)
    q_plain, q_turn = q[..., :dk], rotate_neighbours(q[..., dk:], range(T), dr, m["rot"]["base"])
    src = m.get("kv_from")
    if src is None:
        ckr = h @ t[p + ".dkv"].T
        c = rms_norm(ckr[:, :rank], t[p + ".dkv.norm"], eps)
        kr = rotate_neighbours(ckr[:, None, rank:], range(T), dr, m["rot"]["base"])[:, 0]
        kept[layer] = (c, kr)
    else:
        c, kr = kept[src]
    k_plain = (c @ t[p + ".uk"].T).view(T, H, dk)
    v = (c @ t[p + ".uv"].T).view(T, H, dv)
    k = torch.cat([k_plain, kr[:, None, :].expand(T, H, dr)], dim=-1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = windowed_attention(torch.cat([q_plain, q_turn], dim=-1), k, v, m["scale"], window, sink=False).reshape(T, H * dv)
    return (o * sigmoid(h @ t[p + ".g"].T)) @ t[p + ".o"].T


def dense_feed_forward(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    r = torch.clamp(h @ t[p + ".up"].T, min=0.0)
    return (r * r) @ t[p + ".down"].T


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64,
            stream_after: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``stream_after`` receives the stream after every layer."""
    t = {n: w.to(dtype) for n, w in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][torch.tensor(list(ids), dtype=torch.long)]
    kept: Dict[int, tuple] = {}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}"
        hin = rms_norm(x, t[p + ".norm1"], eps)
        if l["type"] == "attention":
            y = attention_mixer(hin, l["mixer"], t, p + ".mix", eps)
        elif l["type"] == "delta":
            y = delta_mixer(hin, l["mixer"], t, p + ".mix", eps)
        elif l["type"] == "latent_attention":
            y = latent_attention_mixer(hin, l["mixer"], t, p + ".mix", eps, kept, i)
        else:
            raise ValueError(l["type"])
        x = x + t[p + ".ls1"] * y
        if l.get("mlp") is not None:
            x = x + t[p + ".ls2"] * dense_feed_forward(rms_norm(x, t[p + ".norm2"], eps), t, p + ".mlp")
        if stream_after is not None:
            stream_after.append(x.clone())
    logits = rms_norm(x, t["final.norm"], eps) @ t["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits


def generate(cfg: Mapping, tensors: Mapping[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]
