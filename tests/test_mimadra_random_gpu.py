"""Seeded random Mimadra configurations against the plain implementation: layer orders, head counts, key, value and latent
sizes, windows, taps and constants that no hand-written configuration of the other tests has, among them sizes the
tensor-core kernels take (latent rows in multiples of 16 with ranks in multiples of 64, heads of 64 and 128) and sizes only the
CUDA-core kernels take.  Every model runs whole prompts, a prompt then decoded tokens, and an unequal batch decoded together
with requests that end at different times, in both types."""
import numpy as np
import pytest
import torch

from helpers import random_ids, run_schedule
from plain import mimadra_plain as P
from test_mimadra_gpu import _att, _close, _delta, _ff, _lat, _write, make_tensors

pytestmark = pytest.mark.gpu


def random_config(seed):
    r = np.random.default_rng(seed)
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    layers, writers = [], []
    for i in range(int(r.integers(3, 7))):
        kind = pick(["attention", "delta", "latent_attention"])
        ff = pick([None, 136, 200, 256, 320])
        if kind == "attention":
            kv = pick([1, 2, 3])
            dim = pick([32, 48, 64, 80, 128])
            m = _att(kv * pick([1, 2, 4]), kv, dim, pick([32, 64, 96, dim]), float(dim ** -0.5 * r.uniform(0.7, 1.5)),
                     window=pick([None, 5, 40, 64, 100, 136]), rot=(pick([d for d in (8, 16, 32, 64) if d <= dim]), pick([10000.0, 500.0])))
        elif kind == "delta":
            kv = pick([1, 2, 3])
            m = _delta(kv * pick([1, 2, 3]), kv, pick([32, 48, 64, 96, 128]), pick([32, 48, 64, 128]), pick([2, 3, 4, 5]))
        else:
            src = pick(writers) if writers and r.random() < 0.5 else None
            if src is not None:
                sm = layers[src]["mixer"]
                rank, rd, base = sm["kv_rank"], sm["rot_dim"], sm["rot"]["base"]
            else:
                rank, rd, base = pick([64, 72, 96, 128, 192, 256]), pick([8, 16, 32, 48, 64]), pick([10000.0, 250000.0])
                writers.append(i)
            dim = pick([32, 48, 64, 96])
            m = _lat(pick([1, 2, 4, 6, 12, 16]), dim, rd, pick([32, 64, 96, dim]), rank, float((dim + rd) ** -0.5 * r.uniform(0.7, 1.5)),
                     base, window=pick([None, 7, 40, 65, 120]), kv_from=src)
        layers.append({"type": kind, "mixer": m, "mlp": _ff(ff)})
    return {"architecture": "Mimadra", "vocab": int(r.integers(150, 700)), "width": pick([96, 128, 160, 224, 256]),
            "norm": {"eps": pick([1e-5, 1e-6])}, "logit_softcap": pick([30.0, 15.0, 50.0]), "layers": layers}


@pytest.fixture(scope="module", params=[3, 5, 18, 26, 50])     # all but the first with layers that read another layer's rows
def case(request, tmp_path_factory):
    cfg = random_config(request.param)
    t = make_tensors(cfg, 900 + request.param)
    d = _write(tmp_path_factory.mktemp(f"rand{request.param}"), cfg, t, "m")
    V = cfg["vocab"]
    reqs = {"a": random_ids(230, V, request.param * 7 + 1), "b": random_ids(90, V, request.param * 7 + 2), "c": random_ids(31, V, request.param * 7 + 3)}
    want = {k: P.forward(cfg, t, ids).numpy() for k, ids in reqs.items()}
    return d, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(case, dtype):
    from ithaca_b200 import Engine
    d, reqs, want = case
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    schedules = {
        "whole": [[("a", 230)], [("b", 90)], [("c", 31)]],
        "prompt then decode": [[("a", 190)]] + [[("a", 1)] for _ in range(40)],
        "together": [[("a", 170), ("b", 50), ("c", 1)]] + [[("a", 1), ("b", 1), ("c", 1)] for _ in range(30)]
                    + [[("a", 1), ("b", 1)] for _ in range(10)] + [[("a", 1)] for _ in range(20)],
    }
    for label, sched in schedules.items():
        got = run_schedule(eng, reqs, sched)
        for r, lg in got.items():
            assert _close(lg, want[r], dtype), (label, r)
        assert eng.cache.table.n_slots_in_use() == 0
    del eng
    torch.cuda.empty_cache()
