"""Gunenex without a device: the configuration reader, what the model description says, and the plain implementation's
mechanisms against closed forms."""
import copy
import math

import pytest
import torch

from plain import gunenex_plain as P

from ithaca_b200.config import ConfigError, config_from_dict
from ithaca_b200.config.gunenex import GunenexConfig
from ithaca_b200.engine.model import weight_manifest


def _left(heads=4, kv=2, dim=16, vdim=8, scale=0.25, rot=(8, 1000.0)):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


CFG = {
    "architecture": "Gunenex", "vocab": 61, "width": 40, "streams": 2, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 16, "kv_rank": 24, "q_rank": 12, "scale": 0.3},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}},
        {"type": "parallel", "mixer": {"left": _left(), "right": {"heads": 3, "dim": 8}}, "mlp": {"kind": "dense", "ff": 56}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 8, "kv_rank": 24, "q_rank": 8, "scale": 0.2, "kv_from": 0},
         "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}, "mlp": {"kind": "dense", "ff": 32}},
    ],
}


def test_the_description_names_parts_cache_entries_and_tensors():
    arch, cfg = config_from_dict(CFG)
    assert isinstance(cfg, GunenexConfig) and arch.name == "Gunenex"
    spec = cfg.model_spec()
    assert spec.streams == 2 and [b.kind for b in spec.layers] == ["hyper"] * 4
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "parallel", "latent_attention", "gated_delta"]
    assert [(e.cache, e.writes_cache) for e in spec.schedule] == [(0, True), (1, True), (0, False), (2, True)]
    assert [b.kind for b in spec.layers[1].mixer["branches"]] == ["attention", "shift_decay"]
    assert spec.layers[1].mixer["scales"] == [0.5, 0.5]
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.kind == "moe"
    man = weight_manifest(spec)
    assert man["l0.norm1"].shape == () and man["final.norm"].shape == ()
    assert man["l1.hc2.mix"].shape == (2, 2) and man["l1.hc1.in"].shape == (2,)
    assert "l2.hc2.mix" not in man and "l2.mix.dkv" not in man and man["l2.mix.uk"].shape == (48, 24)
    assert man["l1.mix.left.q.b"].shape == (64,) and man["l1.mix.left.sink"].shape == (4,) and man["l1.mix.left.g"].shape == (4, 40)
    assert man["l1.mix.right.mu.w"].shape == (40,) and man["l1.mix.right.u"].shape == (3, 8) and man["l1.mix.right.norm"].shape == (24,)
    assert man["l3.mix.dt_bias"].shape == (32,) and man["l3.mix.a2"].shape[0] == 32 and man["l3.mix.g2"].shape[0] == 48
    assert man["l0.mlp.e4.up"].shape == (24, 40) and "l0.mlp.e0.gate" not in man and man["l0.mlp.router"].shape == (5, 40)
    assert man["l3.mlp.gate"].shape == (32, 40)


def test_ranks_come_from_the_tensors():
    _, cfg = config_from_dict(CFG)
    got = cfg.with_tensor_shapes({"l1.mix.right.w1": (5, 40), "l3.mix.a1": (7, 40), "l3.mix.g1": (3, 40)})
    man = weight_manifest(got.model_spec())
    assert man["l1.mix.right.w2"].shape == (24, 5) and man["l3.mix.a2"].shape == (32, 7) and man["l3.mix.g2"].shape == (48, 3)
    assert config_from_dict(got.to_dict())[1].model_spec() == got.model_spec()          # the written file keeps them


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "attention", "type"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "rot.dims"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 2, "mixer", "kv_rank"), 16, "kv_rank"),
    (("layers", 0, "mlp", "router", "top"), 6, "top"),
    (("layers", 3, "mlp", "kind"), "sparse", "kind"),
    (("layers", 3, "mixer", "conv"), 0, "conv"),
    (("streams",), 0, "streams"),
    (("norm",), None, "norm"),
])
def test_wrong_files_are_refused_with_the_key_named(path, value, word):
    bad = copy.deepcopy(CFG)
    at = bad
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_missing_keys_are_named():
    for path in (("width",), ("streams",), ("layers", 0, "mixer", "q_rank"), ("layers", 1, "mixer", "right"), ("layers", 0, "mlp", "expert")):
        bad = copy.deepcopy(CFG)
        at = bad
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError) as e:
            config_from_dict(bad)
        assert path[-1] in str(e.value)


# ------------------------------------------------------------------------------------------ the plain implementation
def test_plain_sink_takes_the_weight_it_should():
    q = torch.zeros(3, 1, 4, dtype=torch.float64)
    k = torch.zeros(3, 1, 4, dtype=torch.float64)
    v = torch.arange(3, dtype=torch.float64).reshape(3, 1, 1) + 1.0
    out = P.causal_attention(q, k, v, 1.0, torch.tensor([math.log(2.0)], dtype=torch.float64))
    # scores 0: weights 1 / (n + 2) each, the sink holds 2 / (n + 2)
    assert torch.allclose(out[:, 0, 0], torch.tensor([1 / 3, 3 / 4, 6 / 5], dtype=torch.float64))
    free = P.causal_attention(q, k, v, 1.0)
    assert torch.allclose(free[:, 0, 0], torch.tensor([1.0, 1.5, 2.0], dtype=torch.float64))


def test_plain_rotation_turns_pairs_of_halves_and_leaves_the_rest():
    x = torch.zeros(2, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 5] = 7.0
    y = P.rotate_halves(x, [0, 3], 4, 100.0)
    assert torch.allclose(y[0], x[0])
    a = float(torch.tensor(3.0, dtype=torch.float32))
    assert abs(float(y[1, 0, 0]) - math.cos(a)) < 1e-6 and abs(float(y[1, 0, 2]) - math.sin(a)) < 1e-6
    assert float(y[1, 0, 1]) == 0.0 and float(y[1, 0, 5]) == 7.0


def test_plain_channel_delta_rule_closed_forms():
    # decay 1, beta 1, orthonormal keys: the state stores v along k and the read-out returns it
    T, dk, dv = 4, 4, 3
    k = torch.eye(dk, dtype=torch.float64)[:T].reshape(T, 1, dk)
    v = torch.arange(T * dv, dtype=torch.float64).reshape(T, 1, dv) + 1
    one = torch.ones(T, 1, dk, dtype=torch.float64)
    out = P.channel_delta_rule(k.clone(), k, v, torch.ones(T, 1, dtype=torch.float64), one)
    assert torch.allclose(out, v)
    # a decay on channel 0 only: what was written along channel 0 fades, what was written along channel 1 stays
    a = one.clone()
    a[:, 0, 0] = 0.5
    q = torch.zeros(T, 1, dk, dtype=torch.float64)
    q[3, 0, 0] = 1.0
    q[2, 0, 1] = 1.0
    out = P.channel_delta_rule(q, k, v, torch.ones(T, 1, dtype=torch.float64), a)
    assert torch.allclose(out[3, 0], v[0, 0] * 0.5 ** 3) and torch.allclose(out[2, 0], v[1, 0])


def test_plain_token_shift_bonus_and_decay():
    # one head of size 2, width 2, identity projections: the read-out of the first token is the bonus term alone
    d = 2
    eye = torch.eye(d, dtype=torch.float64)
    t = {"p.mu." + s: torch.zeros(d, dtype=torch.float64) for s in "rkvgw"}
    t.update({"p." + s: eye for s in "rkvgo"})
    t.update({"p.w1": torch.zeros(1, d, dtype=torch.float64), "p.w2": torch.zeros(d, 1, dtype=torch.float64),
              "p.w0": torch.full((d,), -50.0, dtype=torch.float64), "p.u": torch.tensor([[2.0, 0.0]], dtype=torch.float64),
              "p.norm": torch.ones(d, dtype=torch.float64)})
    h = torch.tensor([[1.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    out = P.token_shift_mixer(h, {"heads": 1, "dim": 2}, t, "p", 0.0)
    # token 0: o = v * sum_i u_i k_i r_i = [1, 1] * 2 -> normed to [1, 1], gate silu(1)
    g = 1.0 / (1.0 + math.exp(-1.0))
    assert torch.allclose(out[0], torch.tensor([g, g], dtype=torch.float64))
    # token 1 (decay ~ 1): S = k0 v0^T = ones; o = S^T r + v * u_0 k_0 r_0 = [1, 1] + [1, 0] * 2 = [3, 1]
    want = torch.tensor([3.0, 1.0], dtype=torch.float64)
    want = want / torch.sqrt((want * want).mean()) * torch.tensor([g, 0.0], dtype=torch.float64)
    assert torch.allclose(out[1], want)
    # with mu = 1 every projection reads the token before: the first token reads zeros
    t.update({"p.mu." + s: torch.ones(d, dtype=torch.float64) for s in "rkvgw"})
    assert float(P.token_shift_mixer(h, {"heads": 1, "dim": 2}, t, "p", 1e-5)[0].abs().max()) == 0.0


def test_plain_router_weights_multiply_the_input():
    d, ff = 4, 3
    g = torch.Generator().manual_seed(3)
    t = {"p.router": torch.randn(3, d, generator=g, dtype=torch.float64)}
    for e in range(3):
        t[f"p.e{e}.up"], t[f"p.e{e}.down"] = torch.randn(ff, d, generator=g, dtype=torch.float64), torch.randn(d, ff, generator=g, dtype=torch.float64)
    h = torch.randn(5, d, generator=g, dtype=torch.float64)
    chosen = []
    out = P.routed_feed_forward(h, {"router": {"top": 2}}, t, "p", chosen)
    s = P.sigmoid(h @ t["p.router"].T)
    for i in range(5):
        assert chosen[i] == sorted(range(3), key=lambda e: -float(s[i, e]))[:2]
        # the square of relu is homogeneous of degree two: expert(w h) = w^2 expert(h)
        want = sum(float(s[i, e]) ** 2 * (torch.clamp(h[i] @ t[f"p.e{e}.up"].T, min=0) ** 2) @ t[f"p.e{e}.down"].T for e in chosen[i])
        assert torch.allclose(out[i], want)


def test_plain_streams_with_identity_mixing_are_a_plain_residual():
    """Mixing matrix = identity, read and write vectors = first unit vector: stream 0 is an ordinary pre-norm residual
    stream and the others keep the embedding."""
    cfg = copy.deepcopy(CFG)
    cfg["layers"] = cfg["layers"][3:]
    g = torch.Generator().manual_seed(5)
    t = {n: (torch.randn(tuple(r.shape), generator=g) * 0.3).double() for n, r in weight_manifest(config_from_dict(cfg)[1].model_spec()).items()}
    for q in ("hc1", "hc2"):
        t[f"l0.{q}.in"] = torch.tensor([1.0, 0.0], dtype=torch.float64)
        t[f"l0.{q}.out"] = torch.tensor([1.0, 0.0], dtype=torch.float64)
        t[f"l0.{q}.mix"] = torch.eye(2, dtype=torch.float64)
    ids = [3, 9, 27, 1, 40]
    after = []
    P.forward(cfg, t, ids, stream_after=after)
    e = t["embed"][ids]
    x = e + P.channel_delta_mixer(P.rms(e, 1e-5) * t["l0.norm1"], cfg["layers"][0]["mixer"], t, "l0.mix", 1e-5)
    x = x + P.dense_feed_forward(P.rms(x, 1e-5) * t["l0.norm2"], t, "l0.mlp")
    assert torch.allclose(after[0], x + e)
