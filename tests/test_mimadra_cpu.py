"""Mimadra without a device: the configuration reader, the description built from it, the tensors it asks for, which
cache entry a layer gets, and the plain implementation's parts against closed forms."""
import copy
import math

import pytest
import torch

from plain import mimadra_plain as P
from test_mimadra_gpu import CFG_A, CFG_B, CFG_C


def test_layers_sizes_and_constants_come_from_the_file():
    from ithaca_b200.config import config_from_dict, validate_schedule
    from ithaca_b200.engine.model import weight_manifest
    arch, cfg = config_from_dict(CFG_A)
    spec = cfg.model_spec()
    validate_schedule(spec)
    assert arch.name == "Mimadra" and spec.vocab_size == 101 and spec.hidden_size == 64
    m = weight_manifest(spec)
    assert tuple(m["l0.mix.q"].shape) == (3 * (16 + 8), 64) and tuple(m["l0.mix.dkv"].shape) == (40 + 8, 64)
    assert tuple(m["l0.mix.dkv.norm"].shape) == (40,) and tuple(m["l0.mix.uk"].shape) == (3 * 16, 40)
    assert tuple(m["l0.mix.uv"].shape) == (3 * 24, 40) and tuple(m["l0.mix.g"].shape) == (3 * 24, 64) and tuple(m["l0.mix.o"].shape) == (64, 72)
    assert tuple(m["l1.mix.q"].shape) == (2 * 24, 64) and tuple(m["l1.mix.v"].shape) == (4 * 40, 64) and tuple(m["l1.mix.b"].shape) == (4, 64)
    assert tuple(m["l1.mix.q.conv"].shape) == (48, 3) and tuple(m["l1.mix.v.conv"].shape) == (160, 3) and tuple(m["l1.mix.norm"].shape) == (40,)
    assert tuple(m["l1.mix.A_log"].shape) == (4,) and tuple(m["l1.mix.dt_bias"].shape) == (4,) and tuple(m["l4.mix.k.conv"].shape) == (240, 1)
    assert tuple(m["l3.mix.q"].shape) == (6 * 16, 64) and tuple(m["l3.mix.v"].shape) == (2 * 8, 64) and tuple(m["l3.mix.q.norm"].shape) == (16,)
    assert tuple(m["l3.mix.g"].shape) == (6 * 8, 64) and tuple(m["l0.mlp.up"].shape) == (88, 64) and tuple(m["l0.mlp.down"].shape) == (64, 88)
    # a reader has no latent projection of its own; a layer without feed-forward has neither its norm nor its scale
    assert "l2.mix.dkv" not in m and "l2.mix.dkv.norm" not in m and {"l2.mix.uk", "l2.mix.uv", "l2.mix.q", "l2.mix.g"} <= set(m)
    assert not any(n.startswith(("l1.mlp", "l1.norm2", "l1.ls2")) for n in m) and {"l1.norm1", "l1.ls1", "embed", "head", "final.norm"} <= set(m)
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "gated_delta", "latent_attention", "attention", "gated_delta", "attention"]
    assert all(b.kind == "prenorm" for b in spec.layers)
    a = spec.layers[3]
    assert a.mixer["window"] == 33 and a.mixer["sink"] and a.mixer["qk_norm"] == "head" and a.mixer["scale"] == 0.3
    assert a.position["pairing"] == "half" and a.position["rotary_dim"] == 8 and a.position["theta"] == 500.0
    assert spec.layers[5].mixer["window"] is None and spec.layers[0].position["pairing"] == "interleaved"
    assert spec.layers[1].mixer["conv_taps"] == 3 and spec.layers[1].mixer["unit_eps"] == 1e-6 and spec.layers[1].mixer["norm_eps"] == 1e-5
    assert spec.layers[0].feed_forward["activation"] == "relu2" and spec.layers[1].feed_forward is None
    assert spec.head["softcap"] == 8.0 and spec.head.weights["weight"] == "head"
    assert config_from_dict(cfg.to_dict())[1].model_spec() == spec


def test_a_reader_gets_its_writers_cache_entry():
    from ithaca_b200.config import config_from_dict
    s = config_from_dict(CFG_A)[1].model_spec().schedule
    assert [e.layer for e in s] == list(range(6))
    assert [e.cache for e in s] == [0, 1, 0, 2, 3, 4] and [e.writes_cache for e in s] == [True, True, False, True, True, True]
    assert spec_flag(CFG_A, 2) is False and spec_flag(CFG_A, 0) is True
    s = config_from_dict(CFG_C)[1].model_spec().schedule
    assert [e.cache for e in s] == [0, 0, 1, 2] and not s[1].writes_cache


def spec_flag(cfg, layer):
    from ithaca_b200.config import config_from_dict
    return config_from_dict(cfg)[1].model_spec().layers[layer].mixer["own_latent"]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "parallel"), "type"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 4), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 48), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][3]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "mlp.kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_a_wrong_file_is_refused_with_the_key_named(change, word):
    from ithaca_b200.config import ConfigError, config_from_dict
    bad = copy.deepcopy(CFG_A)
    change(bad)
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_what_the_mixers_keep():
    """A latent layer keeps one key/value head of rank + turning part numbers whose values lie in the keys; the delta rule a
    state by parity and, with more than one tap, a ring."""
    from ithaca_b200.cache.cache import KVRequest, StateRequest
    from ithaca_b200.parts.delta import GatedDeltaRule
    from ithaca_b200.parts.latent_attention import LatentAttention
    lat = LatentAttention.__new__(LatentAttention)
    lat.rank, lat.rope_dim, lat.window = 40, 8, 70
    (r,) = lat.cache_requests()
    assert isinstance(r, KVRequest) and (r.n_kv_heads, r.head_dim, r.window, r.values_in_keys) == (1, 48, 70, True)
    d = GatedDeltaRule.__new__(GatedDeltaRule)
    d.n_heads, d.head_dim, d.v_head_dim, d.taps, d.channels = 4, 24, 40, 3, 2 * 2 * 24 + 4 * 40
    st, ring = d.cache_requests()
    assert isinstance(st, StateRequest) and tuple(st.shape) == (2, 4, 40, 24) and tuple(ring.shape) == (3, 256)
    d.taps = 1
    assert len(d.cache_requests()) == 1


# ------------------------------------------------------------------------------------------ the plain implementation
def test_plain_rotations_turn_pairs_by_position_times_frequency():
    x = torch.zeros(2, 1, 8, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                       # halves: dimension 0 pairs with 2 of the first four; the rest pass
    x[:, 0, 6] = 5.0
    y = P.rotate_halves(x, [0, 3], 4, 100.0)
    assert torch.allclose(y[0], x[0]) and abs(float(y[1, 0, 0]) - math.cos(3.0)) < 1e-12 and abs(float(y[1, 0, 2]) - math.sin(3.0)) < 1e-12
    assert float(y[1, 0, 6]) == 5.0 and float(y[1, 0, 1]) == 0.0
    z = torch.zeros(1, 1, 4, dtype=torch.float64)
    z[0, 0, 2] = 1.0                                       # neighbours: dimension 2 pairs with 3, frequency base^(-2/4)
    w = P.rotate_neighbours(z, [7], 4, 100.0)
    a = 7 * 100.0 ** -0.5                                  # the plain angles are formed in 32-bit, as the design has them
    assert abs(float(w[0, 0, 2]) - math.cos(a)) < 1e-6 and abs(float(w[0, 0, 3]) - math.sin(a)) < 1e-6 and float(w[0, 0, 0]) == 0.0


def test_plain_attention_window_and_sink():
    q = torch.zeros(4, 1, 2, dtype=torch.float64)
    k = torch.zeros(4, 1, 2, dtype=torch.float64)
    v = torch.arange(4, dtype=torch.float64).reshape(4, 1, 1) + 1.0
    # all scores 0: ordinary softmax is the mean over the visible keys, the sink adds one to the denominator
    o = P.windowed_attention(q, k, v, 1.0, None, False)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([1.0, 1.5, 2.0, 2.5], dtype=torch.float64))
    o = P.windowed_attention(q, k, v, 1.0, 2, False)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([1.0, 1.5, 2.5, 3.5], dtype=torch.float64))
    o = P.windowed_attention(q, k, v, 1.0, 2, True)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([1.0 / 2, 3.0 / 3, 5.0 / 3, 7.0 / 3], dtype=torch.float64))


def test_plain_convolution_meets_the_current_token_with_the_last_column():
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)
    assert torch.allclose(P.short_convolution(x, w)[:, 0], torch.tensor([1.0, 12.0, 123.0], dtype=torch.float64))


def test_plain_delta_rule_closed_forms():
    """One head, keys along the axes: with step 1 and decay 1 a key's column of the state holds the last value written
    along it (a rewrite replaces, it does not add); with step 1/2 the state moves half way; the decay shrinks what is kept."""
    e0, e1 = torch.tensor([1.0, 0.0], dtype=torch.float64), torch.tensor([0.0, 1.0], dtype=torch.float64)
    k = torch.stack([e0, e1, e0, e0]).reshape(4, 1, 2)
    q = torch.stack([e0, e0, e0, e1]).reshape(4, 1, 2)
    v = torch.tensor([[2.0], [3.0], [5.0], [7.0]], dtype=torch.float64).reshape(4, 1, 1)
    one = torch.ones(4, 1, dtype=torch.float64)
    o = P.gated_delta_rule(q, k, v, one, one)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([2.0, 2.0, 5.0, 3.0], dtype=torch.float64))
    o = P.gated_delta_rule(q, k, v, 0.5 * one, one)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([1.0, 1.0, 3.0, 1.5], dtype=torch.float64))
    o = P.gated_delta_rule(q, k, v, one, 0.5 * one)[:, 0, 0]
    assert torch.allclose(o, torch.tensor([2.0, 1.0, 5.0, 0.75], dtype=torch.float64))


def test_plain_model_is_causal_and_generates():
    from test_mimadra_gpu import make_tensors
    t = make_tensors(CFG_B, 5)
    ids = [3, 9, 27, 14, 60, 2, 8]
    whole = P.forward(CFG_B, t, ids)
    assert whole.shape == (7, CFG_B["vocab"]) and float(whole.abs().max()) <= CFG_B["logit_softcap"]
    assert torch.allclose(P.forward(CFG_B, t, ids[:4]), whole[:4], atol=1e-10)
    out = P.generate(CFG_B, t, ids[:3], 4)
    assert len(out) == 4 and out[0] == int(whole[2].argmax())
