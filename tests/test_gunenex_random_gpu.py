"""Seeded random Gunenex configurations against the plain implementation: layer orders, numbers of streams, head counts, key,
value and latent sizes, ranks, taps, experts and constants that no hand-written configuration of the other tests has, among
them sizes the tensor-core kernels take (latents in multiples of 64, heads of 64 and 128) and sizes only the CUDA-core kernels
take.  Every model runs whole prompts, a prompt then decoded tokens, and an unequal batch decoded together with requests that
end at different times, in both types.

float32: against the plain implementation as it is, every row within the tolerance.  bfloat16: two experts whose scores lie a
few hundredths apart change places under 16-bit operands, and through several routed layers, recurrent states and seven layers
such a token moves many rows behind it.  So the 16-bit run is held against the plain implementation made to use the experts
the library chose for every token (read off the routing kernels' results; which experts are the right ones is what the float32
run and the routing kernels' own tests check), and then the rows must hold as ``rows_hold`` says."""
import numpy as np
import pytest
import torch

from helpers import REL, random_ids, run_schedule
from plain import gunenex_plain as P
from test_gunenex_gpu import _close, _delta, _ff, _lat, _left, _moe, _par, _write, make_tensors, run_tapped, rows_hold

pytestmark = pytest.mark.gpu


def random_config(seed):
    r = np.random.default_rng(seed)
    pick = lambda xs: xs[int(r.integers(0, len(xs)))]
    layers, writers = [], []
    for i in range(int(r.integers(3, 8))):
        kind = pick(["parallel", "channel_delta", "latent_attention"])
        mlp = pick([None, _ff(pick([136, 200, 256])), _moe(pick([48, 64, 104]), pick([2, 4, 7, 16]), 1), _moe(pick([40, 96]), pick([3, 8]), pick([2, 3]))])
        if kind == "parallel":
            kv = pick([1, 2, 3])
            dim = pick([32, 48, 64, 80, 128])
            rot = pick([None] + [(d, pick([10000.0, 250000.0])) for d in (8, 16, 32, 64, 128) if d <= dim])
            m = _par(_left(kv * pick([1, 2, 4]), kv, dim, pick([32, 64, 96, dim]), float(dim ** -0.5 * r.uniform(0.7, 1.5)), rot=rot),
                     pick([1, 2, 5]), pick([16, 32, 48, 64]), rank=pick([None, 8, 20, 64]))
        elif kind == "channel_delta":
            kv = pick([1, 2, 3])
            m = _delta(kv * pick([1, 2, 3]), kv, pick([32, 48, 64, 96, 128]), pick([32, 48, 64, 128]), pick([1, 2, 3, 4, 5]),
                       decay_rank=pick([None, 8, 24, 40]), gate_rank=pick([None, 8, 24, 56]))
        else:
            src = pick(writers) if writers and r.random() < 0.5 else None
            if src is not None:
                rank = layers[src]["mixer"]["kv_rank"]
            else:
                rank = pick([64, 72, 96, 128, 192, 256])
                writers.append(i)
            dim = pick([32, 48, 64, 96])
            m = _lat(pick([1, 2, 4, 6, 12, 16]), dim, pick([32, 64, 96, dim]), rank, pick([24, 64, 96, 160]), float(dim ** -0.5 * r.uniform(0.7, 1.5)),
                     kv_from=src)
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Gunenex", "vocab": int(r.integers(150, 700)), "width": pick([96, 128, 160, 224, 256]),
            "streams": pick([1, 2, 3, 4, 6]), "norm": {"eps": pick([1e-5, 1e-6])}, "layers": layers}


@pytest.fixture(scope="module", params=[2, 7, 13, 26, 32, 55])     # the last four with layers that read another layer's rows
def case(request, tmp_path_factory):
    cfg = random_config(request.param)
    t = make_tensors(cfg, 900 + request.param)
    d = _write(tmp_path_factory.mktemp(f"rand{request.param}"), cfg, t, "m")
    V = cfg["vocab"]
    reqs = {"a": random_ids(230, V, request.param * 7 + 1), "b": random_ids(90, V, request.param * 7 + 2), "c": random_ids(31, V, request.param * 7 + 3)}
    want = {k: P.forward(cfg, t, ids).numpy() for k, ids in reqs.items()}
    return d, cfg, t, reqs, want


def test_random_configuration_with_16_bit_operands(case):
    from ithaca_b200 import Engine
    d, cfg, t, reqs, _ = case
    eng = Engine(d, dtype="bfloat16", max_tokens=1024)
    schedules = {
        "whole": [[("a", 230)], [("b", 90)], [("c", 31)]],
        "together": [[("a", 170), ("b", 50), ("c", 1)]] + [[("a", 1), ("b", 1), ("c", 1)] for _ in range(30)]
                    + [[("a", 1), ("b", 1)] for _ in range(10)] + [[("a", 1)] for _ in range(20)],
    }
    for label, sched in schedules.items():
        got, used = run_tapped(eng, cfg, reqs, sched)
        for r, lg in got.items():
            assert rows_hold(lg, P.forward(cfg, t, reqs[r], forced=used[r]).numpy()), (label, r)
        assert eng.cache.table.n_slots_in_use() == 0
    del eng
    torch.cuda.empty_cache()


def test_random_configuration(case, dtype="float32"):
    from ithaca_b200 import Engine
    d, _, _, reqs, want = case
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
