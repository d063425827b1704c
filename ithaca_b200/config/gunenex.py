"""Typed configuration of the Gunenex decoder, read from ``config.json``.

A Gunenex model lists its layers one by one; every size and constant that can differ between two models of the design
is in the file or in a tensor's shape.  The keys:

* ``vocab``, ``width``, ``streams`` (residual streams per token), ``norm.eps``;
* ``layers``: per layer ``type`` (the mixer: ``parallel``, ``latent_attention`` or ``channel_delta``), ``mixer`` (its sizes and
  constants) and ``mlp`` (``kind: dense`` with ``ff``; ``kind: moe`` with ``expert.ff``, ``router.experts``, ``router.top``; or
  null for none).

A layer is pre-norm over several residual streams: each sublayer reads one combination of the streams through an RMS norm
whose weight is a single number, and its result goes into all streams at once through a small matrix and a vector of the
layer.  ``parallel``: half the sum of two mixers that read the same input, each result first RMS-normed over the width with
a weight of its own: ``left`` a softmax attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot.dims`` leading
dimensions turned in halves with ``rot.base``; biases on the four projections; values normed per head; a learned sink per
head; a gate per head), ``right`` a token-shift time mixing (``heads``, ``dim``; the rank of the decay's first factor is the
first size of its tensor).  ``latent_attention``: keys and values from a latent of ``kv_rank`` values, queries through a
latent of ``q_rank`` values, no positions (``heads``, ``dim``, ``vdim``, ``scale``); with ``kv_from: j`` the layer reads the
rows layer j has written.  ``channel_delta``: the gated delta rule with a decay per head and key channel (``heads``,
``kv_heads`` query/key heads, ``dim``, ``vdim``, ``conv`` taps; the ranks of the decay's and the gate's first factors are
the first sizes of their tensors).  The dense feed-forward is gated with silu; the routed one has sigmoid scores, ungated
experts with the square of relu, and the chosen experts' scores multiply what the experts read.

Tensor names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``, ``norm2``, ``l<i>.hc{1,2}.{in,out,mix}``,
``l<i>.mix.left.{q,k,v,o}`` with ``.b`` for their biases, ``l<i>.mix.left.{sink,g,out}``,
``l<i>.mix.right.{mu.r,mu.k,mu.v,mu.g,mu.w,r,k,v,g,w1,w2,w0,u,norm,o,out}``,
``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}``,
``l<i>.mix.{q,k,v,q.conv,k.conv,v.conv,b,A_log,norm,a1,a2,dt_bias,g1,g2,o}``,
``l<i>.mlp.{gate,up,down}``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, need_float, need_int
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

# no key of the file bounds a sequence's length; this sizes nothing, it only stops a runaway caller
MAX_POSITION = 1 << 20

UNIT_EPS = 1e-6            # inside the root when the delta rule's q and k become unit vectors
BRANCH_WEIGHT = 0.5        # the parallel mixer is half the sum of its two normed branches
TYPES = ("parallel", "latent_attention", "channel_delta")
# ranks that the file does not give: the first size of a low-rank factor.  A model folder's tensors decide; random
# weights take these.
DEFAULT_DECAY_RANK = 32
DEFAULT_GATE_RANK = 32


def _obj(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, found {v!r}")
    return v


def _heads(m: Dict[str, Any], where: str) -> None:
    heads, kv = need_int(m, "heads"), need_int(m, "kv_heads")
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} kv_heads evenly")


@dataclass(frozen=True)
class GunenexConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    streams: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]        # as validated from the file
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Gunenex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GunenexConfig":
        width = need_int(d, "width")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, l in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            m = _obj(l, "mixer", where)
            kind = l.get("type")
            if kind not in TYPES:
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported ({', '.join(TYPES)})")
            if kind == "parallel":
                left, right = _obj(m, "left", where + "mixer."), _obj(m, "right", where + "mixer.")
                _heads(left, where + "mixer.left")
                dim = need_int(left, "dim")
                need_int(left, "vdim"), need_float(left, "scale")
                rot = _obj(left, "rot", where + "mixer.left.", optional=True)
                if rot is not None:
                    dims = need_int(rot, "dims", minimum=0)
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"config.json: {where}mixer.left.rot.dims must be even and at most dim, found {dims}")
                    if need_float(rot, "base") <= 0:
                        raise ConfigError(f"config.json: {where}mixer.left.rot.base must be positive")
                need_int(right, "heads"), need_int(right, "dim")
                if "rank" in right:
                    need_int(right, "rank")
            elif kind == "channel_delta":
                _heads(m, where + "mixer")
                need_int(m, "dim"), need_int(m, "vdim"), need_int(m, "conv")
            else:
                need_int(m, "heads"), need_int(m, "dim"), need_int(m, "vdim"), need_float(m, "scale")
                rank = need_int(m, "kv_rank")
                need_int(m, "q_rank")
                src = m.get("kv_from")
                if src is not None:
                    src = need_int(m, "kv_from", minimum=0)
                    if src >= i or layers[src].get("type") != "latent_attention" or layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from must name an earlier latent_attention layer that "
                                          f"keeps rows of its own, found {src}")
                    if layers[src]["mixer"].get("kv_rank") != rank:
                        raise ConfigError(f"config.json: {where}mixer.kv_rank must equal layer {src}'s")
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      "is not supported (dense, moe, or null for none)")
                if mlp["kind"] == "dense":
                    need_int(mlp, "ff")
                else:
                    need_int(_obj(mlp, "expert", where + "mlp."), "ff")
                    router = _obj(mlp, "router", where + "mlp.")
                    if need_int(router, "top") > need_int(router, "experts"):
                        raise ConfigError(f"config.json: {where}mlp.router.top cannot exceed the number of experts")
        streams = need_int(d, "streams")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=need_int(d, "vocab"), hidden_size=width, streams=streams,
                   norm_eps=need_float(_obj(d, "norm", ""), "eps"), layers=tuple(copy.deepcopy(layers)), raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "streams": self.streams,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "GunenexConfig":
        """The same configuration with the low-rank factors' ranks taken from tensor shapes (name -> shape): the file does
        not state them, the folder's tensors do."""
        layers = copy.deepcopy(list(self.layers))
        for i, l in enumerate(layers):
            p = f"l{i}.mix"
            if l["type"] == "parallel" and f"{p}.right.w1" in shapes:
                l["mixer"]["right"]["rank"] = int(shapes[f"{p}.right.w1"][0])
            elif l["type"] == "channel_delta":
                if f"{p}.a1" in shapes:
                    l["mixer"]["decay_rank"] = int(shapes[f"{p}.a1"][0])
                if f"{p}.g1" in shapes:
                    l["mixer"]["gate_rank"] = int(shapes[f"{p}.g1"][0])
        return GunenexConfig(self.architecture, self.vocab_size, self.hidden_size, self.streams, self.norm_eps, tuple(layers), self.raw)

    # -- the architecture-neutral description --------------------------------------------------
    def _parallel(self, p: str, m: Dict[str, Any]) -> PartSpec:
        d, left, right = self.hidden_size, m["left"], m["right"]
        rot = left.get("rot")
        position = None
        if rot is not None and rot["dims"] > 0:
            position = PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "half", "max_position": MAX_POSITION})
        lw = {r: f"{p}.left.{r}" for r in ("q", "k", "v", "g", "o", "sink")}
        lw.update({f"{r}_bias": f"{p}.left.{r}.b" for r in "qkvo"})
        attention = PartSpec("attention", {
            "hidden_size": d, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "v_head_dim": left["vdim"], "scale": left["scale"], "norm_eps": self.norm_eps, "head_gate": True, "sink": "learned",
            "bias": True, "v_norm": True, "window": None, "position": position}, lw)
        rw = {r: f"{p}.right.{r}" for r in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
        rw.update({f"mu_{s}": f"{p}.right.mu.{s}" for s in ("r", "k", "v", "g", "w")})
        shift = PartSpec("shift_decay", {"hidden_size": d, "n_heads": right["heads"], "head_dim": right["dim"],
                                         "decay_rank": right.get("rank", DEFAULT_DECAY_RANK), "norm_eps": self.norm_eps}, rw)
        return PartSpec("parallel", {"hidden_size": d, "branches": [attention, shift], "scales": [BRANCH_WEIGHT, BRANCH_WEIGHT],
                                     "combine": "norm_sum", "out_norms": [f"{p}.left.out", f"{p}.right.out"],
                                     "norm_eps": self.norm_eps})

    def _delta(self, p: str, m: Dict[str, Any]) -> PartSpec:
        w = {r: f"{p}.{r}" for r in ("q", "k", "v", "o", "b", "a1", "a2", "g1", "g2", "A_log", "dt_bias", "norm")}
        w.update({f"{r}_conv": f"{p}.{r}.conv" for r in "qkv"})
        return PartSpec("gated_delta", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "n_qk_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": self.norm_eps, "unit_eps": UNIT_EPS, "decay": "channel",
            "decay_rank": m.get("decay_rank", DEFAULT_DECAY_RANK), "gate": "sigmoid_lowrank",
            "gate_rank": m.get("gate_rank", DEFAULT_GATE_RANK)}, w)

    def _latent(self, p: str, m: Dict[str, Any]) -> PartSpec:
        w = {r: f"{p}.{r}" for r in ("dq", "uq", "uk", "uv", "o", "dkv")}
        w.update({"dq_norm": f"{p}.dq.norm", "dkv_norm": f"{p}.dkv.norm"})
        return PartSpec("latent_attention", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "head_dim": m["dim"], "rope_dim": 0, "v_head_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"], "norm_eps": self.norm_eps, "window": None,
            "own_latent": m.get("kv_from") is None}, w)

    def _feed_forward(self, p: str, mlp: Dict[str, Any]) -> PartSpec:
        d = self.hidden_size
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": mlp["ff"], "activation": "silu"},
                            {"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"})
        return PartSpec("moe", {"hidden_size": d, "intermediate_size": mlp["expert"]["ff"], "n_experts": mlp["router"]["experts"],
                                "top": mlp["router"]["top"], "score": "sigmoid", "renormalize": False, "expert": "plain",
                                "activation": "relu2", "weight_on": "input"},
                        {"router": f"{p}.router", "up": p + ".e{e}.up", "down": p + ".e{e}.down"})

    def model_spec(self) -> ModelSpec:
        d = self.hidden_size

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": d, "eps": self.norm_eps, "scalar_weight": True}, {"weight": name})

        blocks, schedule = [], []
        entry_of: Dict[int, int] = {}                  # layer -> its cache entry (layers that read another's have none)
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l["mixer"]
            if l["type"] != "latent_attention" or m.get("kv_from") is None:
                entry_of[i] = len(entry_of)
                entry = ScheduleEntry(layer=i, cache=entry_of[i])
            else:
                entry = ScheduleEntry(layer=i, cache=entry_of[int(m["kv_from"])], writes_cache=False)
            if l["type"] == "parallel":
                mixer = self._parallel(p + ".mix", m)
            elif l["type"] == "channel_delta":
                mixer = self._delta(p + ".mix", m)
            else:
                mixer = self._latent(p + ".mix", m)
            ff, norms = None, {"mixer": norm(f"{p}.norm1")}
            params = {"streams": self.streams, "mixer": {r: f"{p}.hc1.{r}" for r in ("in", "out", "mix")}}
            if l.get("mlp") is not None:
                ff = self._feed_forward(p + ".mlp", l["mlp"])
                norms["feed_forward"] = norm(f"{p}.norm2")
                params["feed_forward"] = {r: f"{p}.hc2.{r}" for r in ("in", "out", "mix")}
            blocks.append(BlockSpec(kind="hyper", mixer=mixer, feed_forward=ff, norms=norms, position=None, params=params))
            schedule.append(entry)
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": d}, {"weight": "embed"}),
            layers=tuple(blocks), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": d}, {"weight": "head"}),
            max_position=MAX_POSITION, streams=self.streams,
        )
