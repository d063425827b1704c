"""A plain, slow Gunenex decoder: whole sequences, no cache, one function per mechanism.

Nothing here is shared with the library under test.  It reads ``config.json`` keys from a plain dictionary and
tensors from a plain name -> tensor mapping and computes on the CPU in the dtype it is given (float64 by default,
so that it is the more exact side of a comparison).

The design in this file's notation (T tokens at positions 0 .. T-1, width d, n the number of streams):

* N(x, g) = x / sqrt(mean(x^2) + eps) * g with g ONE number (layer norms and the final norm).
* x_1 = ... = x_n = E[ids].  A sublayer f with the layer's vectors a, b (size n) and matrix M (n x n, [from, to]):
  u = sum_s a_s x_s;  y = f(N(u));  x_t' = sum_s M[s, t] x_s + b_t y for all t at once.  A layer is its mixer, then
  its feed-forward, both so.  After the last layer x = sum_s x_s, logits = W N(x).
* mixer ``parallel``: half of [R(left(h)) * w_left + R(right(h)) * w_right], R the RMS norm over the width.
  left: softmax attention, H heads over G key/value heads, projections with biases; the leading r dimensions of
  every q and k head turn in pairs (i, i + r/2) by p * base^(-2i/r); every value head is divided by its root mean
  square; scores (q . k) * c over all positions up to the own; the softmax's denominator has one more term
  exp(sink_h); head h times sigmoid((Wg h)_h); output projection with bias.
  right: with h' the input one position earlier (zero at position 0), m_s = h + (h' - h) * mu_s for s in r, k, v, g, w;
  r, k, v = W m (H heads of size D); gate = silu(Wg m_g); w = exp(-exp(W2 tanh(W1 m_w) + w0)) per head and channel;
  per head o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T; every head's o divided by its root
  mean square, all heads times a weight of size H D, times the gate; output projection.
* mixer ``latent_attention``: cq = RMS(Wdq h) * wq, q = Wuq cq; c = RMS(Wdkv h) * wc; per head k = Wuk c, v = Wuv c;
  scores (q . k) * c over all positions up to the own; ordinary softmax; output projection.  No positions.  A layer
  with ``kv_from: j`` has no Wdkv and uses layer j's c.
* mixer ``channel_delta``: q, k (G heads of size D) and v (H heads of size Dv) pass a causal convolution over time
  per channel and silu; q and k become unit vectors per head (1e-6 inside the root), q times D^(-1/2);
  beta = sigmoid(Wb h) per head; decay a = exp(-exp(A_log_h) * softplus(Wa2 (Wa1 h) + dt_bias)) per head AND key
  channel; per head S <- diag(a) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; o RMS-normed over Dv with a
  weight of that size, times sigmoid(Wg2 (Wg1 h)); output projection.
* feed-forward ``dense``: Wdown (silu(Wgate h) * (Wup h)).  ``moe``: s = sigmoid(Wrouter h); the ``top`` experts of
  largest s; output sum_e expert_e(s_e h) with expert(z) = Wdown relu(Wup z)^2.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

UNIT_EPS = 1e-6


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotate_halves(x: torch.Tensor, positions: Sequence[int], r: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: the pair (i, i + r/2) of every head's leading r dimensions turns by p * base^(-2i/r).
    Positions and angles are 32-bit numbers in the design: frequency and product are rounded to float32."""
    y = x.clone()
    p = torch.tensor(list(positions), dtype=torch.float32)[:, None]
    f = torch.tensor([float(base) ** (-2.0 * i / r) for i in range(r // 2)], dtype=torch.float64).to(torch.float32)[None, :]
    a = (p * f).to(x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :r // 2], x[..., r // 2:r]
    y[..., :r // 2] = u * c - v * s
    y[..., r // 2:r] = v * c + u * s
    return y


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; query i sees keys 0 .. i.  ``sink`` [H]: one more
    term exp(sink_h) in the denominator, with no value behind it."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, h]) * scale
            m = float(s.max()) if sink is None else max(float(s.max()), float(sink[h]))
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else math.exp(float(sink[h]) - m))
            out[i, h] = (e / den) @ v[:i + 1, g]
    return out


def sink_attention_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + ".q"].T + t[p + ".q.b"]).view(T, H, dk)
    k = (h @ t[p + ".k"].T + t[p + ".k.b"]).view(T, G, dk)
    v = (h @ t[p + ".v"].T + t[p + ".v.b"]).view(T, G, dv)
    rot = m.get("rot")
    if rot is not None and rot["dims"] > 0:
        q = rotate_halves(q, range(T), rot["dims"], rot["base"])
        k = rotate_halves(k, range(T), rot["dims"], rot["base"])
    v = rms(v, eps)
    o = causal_attention(q, k, v, m["scale"], t[p + ".sink"])
    o = o * sigmoid(h @ t[p + ".g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ t[p + ".o"].T + t[p + ".o.b"]


def token_shift_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mixed(s):
        return h + (before - h) * t[p + ".mu." + s]

    r = (mixed("r") @ t[p + ".r"].T).view(T, H, D)
    k = (mixed("k") @ t[p + ".k"].T).view(T, H, D)
    v = (mixed("v") @ t[p + ".v"].T).view(T, H, D)
    gate = silu(mixed("g") @ t[p + ".g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mixed("w") @ t[p + ".w1"].T) @ t[p + ".w2"].T + t[p + ".w0"])).view(T, H, D)
    u = t[p + ".u"]
    out = torch.zeros((T, H, D), dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros((D, D), dtype=h.dtype)
        for i in range(T):
            kv = torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = (S + u[hd][:, None] * kv).T @ r[i, hd]
            S = w[i, hd][:, None] * S + kv
    o = rms(out, eps).reshape(T, H * D) * t[p + ".norm"] * gate
    return o @ t[p + ".o"].T


def parallel_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    a = sink_attention_mixer(h, m["left"], t, p + ".left", eps)
    b = token_shift_mixer(h, m["right"], t, p + ".right", eps)
    return 0.5 * (rms(a, eps) * t[p + ".left.out"] + rms(b, eps) * t[p + ".right.out"])


def latent_attention_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float,
                           kept: Dict[int, torch.Tensor], layer: int) -> torch.Tensor:
    """``kept``: layer -> latent [T, kv_rank] of the layers that made their own."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = ((rms(h @ t[p + ".dq"].T, eps) * t[p + ".dq.norm"]) @ t[p + ".uq"].T).view(T, H, dk)
    src = m.get("kv_from")
    if src is None:
        c = kept[layer] = rms(h @ t[p + ".dkv"].T, eps) * t[p + ".dkv.norm"]
    else:
        c = kept[src]
    k = (c @ t[p + ".uk"].T).view(T, H, dk)
    v = (c @ t[p + ".uv"].T).view(T, H, dv)
    return causal_attention(q, k, v, m["scale"]).reshape(T, H * dv) @ t[p + ".o"].T


def short_convolution(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]: y[p, c] = sum_j w[c, j] x[p - (taps - 1 - j), c], zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * w[:, j]
    return y


def channel_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """q, k, a [T, H, dk] (already per value head), v [T, H, dv], beta [T, H] -> [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for h in range(H):
        S = torch.zeros((dk, dv), dtype=q.dtype)
        for i in range(T):
            S = a[i, h][:, None] * S
            u = beta[i, h] * (v[i, h] - S.T @ k[i, h])
            S = S + torch.outer(k[i, h], u)
            out[i, h] = S.T @ q[i, h]
    return out


def channel_delta_mixer(h: torch.Tensor, m: Mapping, t: Mapping[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ t[p + ".q"].T, t[p + ".q.conv"])).view(T, G, dk)
    k = silu(short_convolution(h @ t[p + ".k"].T, t[p + ".k.conv"])).view(T, G, dk)
    v = silu(short_convolution(h @ t[p + ".v"].T, t[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = sigmoid(h @ t[p + ".b"].T)
    step = softplus((h @ t[p + ".a1"].T) @ t[p + ".a2"].T + t[p + ".dt_bias"]).view(T, H, dk)
    a = torch.exp(-torch.exp(t[p + ".A_log"])[None, :, None] * step)
    o = rms(channel_delta_rule(q, k, v, beta, a), eps) * t[p + ".norm"]
    gate = sigmoid((h @ t[p + ".g1"].T) @ t[p + ".g2"].T)
    return (o.reshape(T, H * dv) * gate) @ t[p + ".o"].T


def dense_feed_forward(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ t[p + ".gate"].T) * (h @ t[p + ".up"].T)) @ t[p + ".down"].T


def routed_feed_forward(h: torch.Tensor, mlp: Mapping, t: Mapping[str, torch.Tensor], p: str,
                        chosen_out: Optional[List] = None, forced: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
    """``forced``: per token the experts to use instead of the ones with the largest scores (for a comparison with 16-bit
    arithmetic, where two scores a hair apart may change places; the weights are this function's own scores all the same)."""
    top = mlp["router"]["top"]
    s = sigmoid(h @ t[p + ".router"].T)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        best = sorted(range(s.shape[1]), key=lambda e: (-float(s[i, e]), e))[:top] if forced is None else list(forced[i])
        if chosen_out is not None:
            chosen_out.append(best)
        for e in best:
            z = torch.clamp((s[i, e] * h[i]) @ t[f"{p}.e{e}.up"].T, min=0.0)
            out[i] += (z * z) @ t[f"{p}.e{e}.down"].T
    return out


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64,
            stream_after: Optional[List[torch.Tensor]] = None, forced: Optional[Mapping[int, Sequence[Sequence[int]]]] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``stream_after`` receives the sum of the streams after every layer.
    ``forced``: layer -> per token the experts its routed feed-forward is to use."""
    t = {n: w.to(dtype) if w.dtype.is_floating_point else w for n, w in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    n = int(cfg["streams"])
    e = t["embed"][torch.tensor(list(ids), dtype=torch.long)]
    xs = [e.clone() for _ in range(n)]
    kept: Dict[int, torch.Tensor] = {}

    def sublayer(xs, hc, g, f):
        u = sum(t[hc + ".in"][s] * xs[s] for s in range(n))
        y = f(rms(u, eps) * t[g])
        return [sum(t[hc + ".mix"][s, k] * xs[s] for s in range(n)) + t[hc + ".out"][k] * y for k in range(n)]

    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}", l["mixer"]
        if l["type"] == "parallel":
            f = lambda hin: parallel_mixer(hin, m, t, p + ".mix", eps)
        elif l["type"] == "latent_attention":
            f = lambda hin: latent_attention_mixer(hin, m, t, p + ".mix", eps, kept, i)
        elif l["type"] == "channel_delta":
            f = lambda hin: channel_delta_mixer(hin, m, t, p + ".mix", eps)
        else:
            raise ValueError(l["type"])
        xs = sublayer(xs, p + ".hc1", p + ".norm1", f)
        mlp = l.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                g = lambda hin: dense_feed_forward(hin, t, p + ".mlp")
            else:
                g = lambda hin: routed_feed_forward(hin, mlp, t, p + ".mlp", forced=None if forced is None else forced[i])
            xs = sublayer(xs, p + ".hc2", p + ".norm2", g)
        if stream_after is not None:
            stream_after.append(sum(xs).clone())
    return (rms(sum(xs), eps) * t["final.norm"]) @ t["head"].T


def generate(cfg: Mapping, tensors: Mapping[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(cfg, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]
