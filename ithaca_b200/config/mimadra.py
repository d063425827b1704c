"""Typed configuration of the Mimadra decoder, read from ``config.json``.

A Mimadra model lists its layers one by one; every size and constant that can differ between two models of the design
is in the file.  The keys:

* ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``;
* ``layers``: per layer ``type`` (the mixer: ``attention``, ``delta`` or ``latent_attention``), ``mixer`` (its sizes and
  constants) and ``mlp`` (``kind: dense`` with ``ff``, or null for none).

A layer is pre-norm with a per-channel scale on what each sublayer adds to the stream.  ``attention``: grouped heads
(``heads``, ``kv_heads``, ``dim``, ``vdim``), q and k normed per head, the leading ``rot.dims`` dimensions turned in halves
(``rot.base``), ``scale``, a window ``mask.size``, a sink in the softmax and a gate per value.  ``delta``: the gated delta
rule (``heads``, ``kv_heads`` query/key heads, ``dim``, ``vdim``, ``conv`` taps).  ``latent_attention``: keys and values from a
latent of ``kv_rank`` values and a shared turning key part of ``rot_dim`` (``heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``,
``rot.base``, neighbouring pairs); with ``kv_from: j`` the layer reads the rows layer j has written.  The feed-forward is
ungated with the square of relu.  The output matrix is the model's own; logits are capped.

Tensor names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``, ``norm2``, ``ls1``, ``ls2``,
``l<i>.mix.{q,k,v,g,o}``, ``l<i>.mix.{q.norm,k.norm}``, ``l<i>.mix.{q.conv,k.conv,v.conv,b,a,A_log,dt_bias,norm}``,
``l<i>.mix.{dkv,dkv.norm,uk,uv}``, ``l<i>.mlp.{up,down}``.
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
TYPES = ("attention", "delta", "latent_attention")


def _obj(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, found {v!r}")
    return v


def _window(m: Dict[str, Any], where: str) -> Optional[int]:
    mask = _obj(m, "mask", where, optional=True)
    return None if mask is None else need_int(mask, "size")


def _rot(m: Dict[str, Any], where: str, most: int, optional: bool) -> Optional[Dict[str, Any]]:
    rot = _obj(m, "rot", where, optional=optional)
    if rot is not None:
        dims = need_int(rot, "dims")
        if dims % 2 or dims > most:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most {most}, found {dims}")
        if need_float(rot, "base") <= 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
    return rot


@dataclass(frozen=True)
class MimadraConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_softcap: float
    layers: Tuple[Dict[str, Any], ...]        # as validated from the file
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Mimadra"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MimadraConfig":
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
            heads, dim = need_int(m, "heads"), need_int(m, "dim")
            need_int(m, "vdim")
            if kind in ("attention", "delta"):
                kv = need_int(m, "kv_heads")
                if heads % kv:
                    raise ConfigError(f"config.json: {where}mixer: {heads} heads cannot share {kv} kv_heads evenly")
            if kind == "attention":
                need_float(m, "scale"), _window(m, where + "mixer."), _rot(m, where + "mixer.", dim, optional=True)
            elif kind == "delta":
                need_int(m, "conv")
            else:
                need_float(m, "scale"), _window(m, where + "mixer.")
                rank, rd = need_int(m, "kv_rank"), need_int(m, "rot_dim")
                rot = _rot(m, where + "mixer.", rd, optional=False)
                if rot["dims"] != rd:
                    raise ConfigError(f"config.json: {where}mixer.rot.dims must equal rot_dim ({rd}), found {rot['dims']}")
                src = m.get("kv_from")
                if src is not None:
                    src = need_int(m, "kv_from", minimum=0)
                    if src >= i or layers[src].get("type") != "latent_attention" or layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from must name an earlier latent_attention layer that "
                                          f"keeps rows of its own, found {src}")
                    sm = layers[src]["mixer"]
                    if (sm.get("kv_rank"), sm.get("rot_dim"), sm.get("rot")) != (rank, rd, m.get("rot")):
                        raise ConfigError(f"config.json: {where}mixer: kv_rank, rot_dim and rot must equal layer {src}'s")
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      "is not supported (dense, or null for none)")
                need_int(mlp, "ff")
        cap = need_float(d, "logit_softcap", 0.0)
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' cannot be negative")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=need_int(d, "vocab"), hidden_size=width,
                   norm_eps=need_float(_obj(d, "norm", ""), "eps"), logit_softcap=cap, layers=tuple(copy.deepcopy(layers)),
                   raw=copy.deepcopy(d))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap, "layers": copy.deepcopy(list(self.layers))}

    # -- the architecture-neutral description --------------------------------------------------
    def _attention(self, p: str, m: Dict[str, Any]):
        rot = m.get("rot")
        position = None if rot is None else PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "half",
                                                                 "max_position": MAX_POSITION})
        w = {r: f"{p}.mix.{r}" for r in "qkvgo"}
        w.update({"q_norm": f"{p}.mix.q.norm", "k_norm": f"{p}.mix.k.norm"})
        mask = m.get("mask")
        return PartSpec("attention", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "scale": m["scale"], "qk_norm": "head", "norm_eps": self.norm_eps, "head_gate": "wide",
            "sink": True, "window": None if mask is None else mask["size"]}, w), position

    def _delta(self, p: str, m: Dict[str, Any]) -> PartSpec:
        w = {r: f"{p}.mix.{r}" for r in ("q", "k", "v", "g", "o", "b", "a", "A_log", "dt_bias", "norm")}
        w.update({f"{r}_conv": f"{p}.mix.{r}.conv" for r in "qkv"})
        return PartSpec("gated_delta", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "n_qk_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": self.norm_eps, "unit_eps": UNIT_EPS}, w)

    def _latent(self, p: str, m: Dict[str, Any]):
        position = PartSpec("rotary", {"rotary_dim": m["rot_dim"], "theta": m["rot"]["base"], "pairing": "interleaved",
                                       "max_position": MAX_POSITION})
        w = {r: f"{p}.mix.{r}" for r in ("q", "uk", "uv", "g", "o", "dkv")}
        w["dkv_norm"] = f"{p}.mix.dkv.norm"
        mask = m.get("mask")
        return PartSpec("latent_attention", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "head_dim": m["dim"], "rope_dim": m["rot_dim"],
            "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": self.norm_eps, "head_gate": "wide",
            "window": None if mask is None else mask["size"], "own_latent": m.get("kv_from") is None}, w), position

    def model_spec(self) -> ModelSpec:
        d = self.hidden_size

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": d, "eps": self.norm_eps}, {"weight": name})

        blocks, schedule = [], []
        entry_of: Dict[int, int] = {}                  # layer -> its cache entry (layers that read another's have none)
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l["mixer"]
            position = None
            if l["type"] != "latent_attention" or m.get("kv_from") is None:
                entry_of[i] = len(entry_of)
                entry = ScheduleEntry(layer=i, cache=entry_of[i])
            if l["type"] == "attention":
                mixer, position = self._attention(p, m)
            elif l["type"] == "delta":
                mixer = self._delta(p, m)
            else:
                mixer, position = self._latent(p, m)
                if m.get("kv_from") is not None:
                    entry = ScheduleEntry(layer=i, cache=entry_of[int(m["kv_from"])], writes_cache=False)
            ff, norms, scales = None, {"mixer": norm(f"{p}.norm1")}, {"mixer": f"{p}.ls1"}
            if l.get("mlp") is not None:
                ff = PartSpec("mlp", {"hidden_size": d, "intermediate_size": l["mlp"]["ff"], "activation": "relu2"},
                              {"up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
                norms["feed_forward"] = norm(f"{p}.norm2")
                scales["feed_forward"] = f"{p}.ls2"
            blocks.append(BlockSpec(kind="prenorm", mixer=mixer, feed_forward=ff, norms=norms, position=position,
                                    params={"layer_scale": scales}))
            schedule.append(entry)
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": d}, {"weight": "embed"}),
            layers=tuple(blocks), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": d, "softcap": self.logit_softcap},
                          {"weight": "head"}),
            max_position=MAX_POSITION,
        )
