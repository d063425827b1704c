"""The Mimadra decoder and its mechanisms against the plain implementation (tests/plain/mimadra_plain.py).

Small configurations with weights made here.  Per mechanism: the kernel against the plain function, also across several
steps where it carries a state, and a one-layer model of each mixer.  Whole models: prompts against token-by-token
decoding, portions down to two tokens, batches of unequal requests against each alone, slots, pages and states that are
used again, long decoding, and greedy generation through the engine's own loop.  Where random weights would hide a fault
(a key at a window's edge, a far key, a sink, a state that was lost on the way), the weights are made so that one token
decides the result.
"""
import json
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from helpers import REL, random_ids, rel_err, run_schedule
from plain import mimadra_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _att(heads, kv, dim, vdim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def _lat(heads, dim, rd, vdim, rank, scale, base, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rd, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"dims": rd, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


# unlike layers in an unusual order: a latent layer first, read again two layers later through a WIDER window than its
# writer's; windows that end inside a page and span more than one; value sizes unlike key sizes; a part of the head turned and
# the whole head; no window at all; layers without feed-forward; a delta layer whose key size is no multiple of its row
# blocks, one tap and three
CFG_A = {
    "architecture": "Mimadra", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "layers": [
        {"type": "latent_attention", "mixer": _lat(3, 16, 8, 24, 40, 0.2, 1000.0, window=70), "mlp": _ff(88)},
        {"type": "delta", "mixer": _delta(4, 2, 24, 40, 3), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(2, 8, 8, 16, 40, 0.3, 1000.0, window=100, kv_from=0), "mlp": _ff(40)},
        {"type": "attention", "mixer": _att(6, 2, 16, 8, 0.3, window=33, rot=(8, 500.0)), "mlp": _ff(72)},
        {"type": "delta", "mixer": _delta(3, 3, 80, 16, 1), "mlp": _ff(56)},
        {"type": "attention", "mixer": _att(2, 2, 32, 32, 0.2, rot=(32, 10000.0)), "mlp": None},
    ],
}
# one head everywhere, no rotation in the attention, a window of two, a turning part of one pair, four taps, no window on the
# latent layer, hardly a cap on the logits
CFG_B = {
    "architecture": "Mimadra", "vocab": 67, "width": 48, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
    "layers": [
        {"type": "attention", "mixer": _att(1, 1, 64, 16, 0.15, window=2), "mlp": _ff(56)},
        {"type": "delta", "mixer": _delta(1, 1, 16, 32, 4), "mlp": _ff(64)},
        {"type": "latent_attention", "mixer": _lat(1, 32, 2, 8, 16, 0.25, 50.0), "mlp": None},
    ],
}
# latents wide enough for the kernel whose tile rows are the heads (bfloat16): five heads (rows of two tokens share a tile),
# a reader with forty heads (more than one tile of heads) and a window of its own, a latent layer without a window
CFG_C = {
    "architecture": "Mimadra", "vocab": 89, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "layers": [
        {"type": "latent_attention", "mixer": _lat(5, 16, 16, 24, 64, 0.2, 1000.0, window=70), "mlp": _ff(72)},
        {"type": "latent_attention", "mixer": _lat(40, 8, 16, 8, 64, 0.3, 1000.0, window=129, kv_from=0), "mlp": None},
        {"type": "delta", "mixer": _delta(2, 1, 16, 32, 2), "mlp": _ff(48)},
        {"type": "latent_attention", "mixer": _lat(2, 32, 32, 16, 128, 0.15, 10000.0), "mlp": _ff(40)},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def make_tensors(cfg, seed):
    """Weights by name with the shapes the library asks for; scales chosen so that activations are of order one."""
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, req in weight_manifest(config_from_dict(cfg)[1].model_spec()).items():
        shape = tuple(req.shape)
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith((".ls1", ".ls2")):
            t = 0.7 + 0.2 * r
        elif "norm" in name:
            t = 1.0 + 0.1 * r
        elif name.endswith(".conv"):
            t = 0.6 * r
        elif name.endswith(".dt_bias"):
            t = 0.5 * r - 1.0
        elif name.endswith(".A_log"):
            t = 0.5 * r - 0.5
        else:
            t = r * (1.2 / shape[1] ** 0.5)
        out[name] = t.bfloat16()
    return out


def _write(tmp, cfg, tensors, tag):
    from ithaca_b200.weights.safetensors_io import write_file
    d = os.path.join(str(tmp), tag)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("mimadra")
    out = {}
    for i, (n, c) in enumerate(CONFIGS.items()):
        t = make_tensors(c, 50 + i)
        out[n] = (_write(root, c, t, n), t)
    return out


def _close(got, want, dtype):
    """float32: every logit within the tolerance.  bfloat16: the median row must hold the tolerance and none may pass two and
    a half times it (a wrong key or a lost state moves a row by tens of hundredths, see the needle tests)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.all(np.isfinite(got))
    rows = np.abs(got - want).reshape(-1, want.shape[-1]).max(-1) / max(np.abs(want).max(), 1e-30)
    if dtype == "float32":
        return bool(rows.max() < REL[dtype])
    return bool(np.median(rows) < REL[dtype] and rows.max() < 2.5 * REL[dtype])


def _plain(cfg, t, ids):
    return P.forward(cfg, t, ids).numpy()


def _ctx(lo, hi, slots):
    """The device arrays of a step in which sequence b brings positions lo[b] .. hi[b] - 1."""
    new = [h - l for l, h in zip(lo, hi)]
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    return SimpleNamespace(
        n_seqs=len(lo), is_decode=all(n == 1 for n in new), slots=i32(slots), cu_seqlens=i32(np.concatenate([[0], np.cumsum(new)])),
        kv_lens=i32(hi), token_seq=i32(np.repeat(np.arange(len(lo)), new)),
        token_pos=i32(np.concatenate([np.arange(l, h) for l, h in zip(lo, hi)]) if sum(new) else []))


STEPS = [([0, 0, 0], [67, 1, 60]), ([67, 1, 60], [70, 2, 131]), ([70, 2, 131], [71, 3, 132]), ([71, 3, 132], [72, 4, 133])]
TOTAL = [72, 4, 133]


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("d", [48, 256, 1100, 8200])
def test_scaled_add_with_the_next_norm(d):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(d)
    y, res = torch.randn(7, d, generator=g) * 3, torch.randn(7, d, generator=g)
    w, ls = torch.randn(d, generator=g), torch.randn(d, generator=g)
    new = res.double() + ls.double() * y.double()
    r = res.clone().to(DEV)
    xn = ops.scale_add_norm(y.to(DEV), ls.to(DEV), r, w.to(DEV), 1e-5, torch.float32)
    assert rel_err(r.cpu().numpy(), new.numpy()) < 1e-6
    assert rel_err(xn.cpu().numpy(), P.rms_norm(new, w, 1e-5).numpy()) < 3e-6
    r2 = res.clone().to(DEV)
    assert ops.scale_add_norm(y.to(DEV), None, r2) is None                       # no scale, no norm: a plain add
    assert rel_err(r2.cpu().numpy(), (res.double() + y.double()).numpy()) < 1e-6
    r3 = res.clone().to(DEV)
    xb = ops.scale_add_norm(y.to(DEV), ls.to(DEV), r3, w.to(DEV), 1e-5, torch.bfloat16)
    assert torch.equal(r3, r) and rel_err(xb.float().cpu().numpy(), P.rms_norm(new, w, 1e-5).numpy()) < 8e-3


def test_ungated_activations():
    from ithaca_b200.csrc import ops
    x = torch.linspace(-6, 6, 1001).reshape(7, 143).contiguous()
    got = ops.plain_act(x.to(DEV), torch.float32, "relu2").cpu()
    assert rel_err(got.numpy(), (torch.clamp(x.double(), min=0) ** 2).numpy()) < 1e-6
    assert float(got[x < 0].abs().max()) == 0.0
    z = x.double()
    gelu = 0.5 * z * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3)))
    assert rel_err(ops.plain_act(x.to(DEV), torch.float32, "gelu_tanh").cpu().numpy(), gelu.numpy()) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,hdv,rot", [(6, 2, 16, 8, 8), (2, 2, 32, 32, 32), (3, 1, 24, 40, 0), (1, 1, 64, 16, 16), (9, 9, 40, 8, 12)])
def test_per_head_norm_rotation_append_kernel(dtype, nh, nkv, hd, hdv, rot):
    """q and k normed head by head with one shared weight of a head's size, the leading dimensions turned in halves, k and v
    into scrambled pages; the inputs are a column range of a wider matrix."""
    from test_kernels_gpu import Paged
    from ithaca_b200.csrc import ops
    lens, new = [70, 5, 130], [3, 5, 66]
    T, pad = sum(new), 7
    g = torch.Generator().manual_seed(hd + rot)
    wide = torch.randn(T, pad + (nh + nkv) * hd + nkv * hdv + 3, generator=g)
    qw, kw = torch.randn(hd, generator=g), torch.randn(hd, generator=g)
    pk, pv = Paged(lens, nkv, hd, dtype, 5), Paged(lens, nkv, hdv, dtype, 5)
    k_d, v_d, tab = pk.dev()[0], pv.dev()[0], pk.dev()[2]
    seq = torch.from_numpy(np.repeat(np.arange(3), new).astype(np.int32)).to(DEV)
    posn = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)])
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    freqs = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV) if rot else None
    ops.norm_rope_append(wide.to(DEV)[:, pad:], 0, nh * hd, (nh + nkv) * hd, qw.to(DEV), kw.to(DEV), 1e-5, q_out, k_d, v_d, seq,
                         torch.from_numpy(posn.astype(np.int32)).to(DEV), tab, freqs, 1.0, nh, rot, 0, True, status, per_head=True)
    assert status.item() == 0
    x = wide[:, pad:].double()
    q = P.rms_norm(x[:, :nh * hd].reshape(T, nh, hd), qw, 1e-5)
    k = P.rms_norm(x[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), kw, 1e-5)
    v = x[:, (nh + nkv) * hd:(nh + nkv) * hd + nkv * hdv]
    if rot:
        q, k = P.rotate_halves(q, posn, rot, 300.0), P.rotate_halves(k, posn, rot, 300.0)
    tol = 5e-6 if dtype == torch.float32 else 8e-3
    assert rel_err(q_out.float().cpu().numpy(), q.reshape(T, -1).numpy()) < tol
    t = 0
    for b, (l, n) in enumerate(zip(lens, new)):
        for j in range(l - n, l):
            kk, vv = k_d.cpu()[pk.table[b, j // 64], :, j % 64].float(), v_d.cpu()[pk.table[b, j // 64], :, j % 64].float()
            assert rel_err(kk.numpy(), k[t].numpy()) < tol and rel_err(vv.numpy(), v[t].reshape(nkv, hdv).numpy()) < tol
            t += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,hdv,window,sink", [(4, 2, 16, 8, 33, True), (2, 2, 32, 32, 0, True), (3, 1, 48, 24, 70, True),
                                                       (2, 1, 64, 64, 128, True), (2, 2, 16, 16, 5, False)])
def test_attention_with_a_sink(dtype, nh, nkv, hd, hdv, window, sink):
    """Queries of a portion and of single tokens over scrambled pages: the weights are exp(s) / (1 + sum exp(s)).  Scores are
    made small and large so that the sink takes most of the weight for some queries and next to none for others."""
    from test_kernels_gpu import Paged
    from ithaca_b200.csrc import ops
    lens, new = [200, 1, 131], [70, 1, 1]
    g = torch.Generator().manual_seed(hd + window)
    ks = [torch.randn(l, nkv, hd, generator=g) for l in lens]
    vs = [torch.randn(l, nkv, hdv, generator=g) for l in lens]
    qs = [torch.randn(l, nh, hd, generator=g) * torch.linspace(0.05, 3.0, l)[:, None, None] for l in lens]
    pk, pv = Paged(lens, nkv, hd, dtype, 3), Paged(lens, nkv, hdv, dtype, 3)
    pk.fill(ks, ks)
    pv.fill(vs, vs)
    k_d, v_d, tab = pk.dev()[0], pv.dev()[0], pk.dev()[2]
    seq = torch.from_numpy(np.repeat(np.arange(3), new).astype(np.int32)).to(DEV)
    posn = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)]).astype(np.int32)
    q = torch.cat([a[l - n:] for a, l, n in zip(qs, lens, new)]).reshape(sum(new), nh * hd).to(dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.attention_simt(q.to(DEV), k_d, v_d, seq, torch.from_numpy(posn).to(DEV), tab, nh, 0.3, window, status, sink=sink)
    assert status.item() == 0
    rt = lambda a: a.to(dtype).double()
    want = torch.cat([P.windowed_attention(rt(qs[b]), rt(ks[b]), rt(vs[b]), 0.3, window or None, sink)[l - n:]
                      for b, (l, n) in enumerate(zip(lens, new))])
    assert rel_err(out.float().cpu().numpy(), want.reshape(sum(new), -1).numpy()) < (3e-6 if dtype == torch.float32 else 8e-3)
    if sink:
        free = torch.cat([P.windowed_attention(rt(qs[b]), rt(ks[b]), rt(vs[b]), 0.3, window or None, False)[l - n:]
                          for b, (l, n) in enumerate(zip(lens, new))])
        assert rel_err(free.numpy(), want.numpy()) > 0.1                     # the sink matters here


@pytest.mark.parametrize("nh,nkv,hd,kind,window", [(4, 2, 16, "mma", 33), (2, 2, 32, "mma", 0), (4, 2, 64, "tc", 70), (8, 2, 128, "tc", 130),
                                                   (2, 1, 128, "mma", 64), (3, 3, 64, "tc", 0)])
def test_tensor_core_attention_with_a_sink(nh, nkv, hd, kind, window):
    """The bfloat16 kernels, prompts' portions (both kernels) and single tokens (chunks of one and of four pages): the sink
    joins the running maximum and sum once, however many pages and chunks a query's keys span."""
    from test_kernels_gpu import Paged
    from ithaca_b200.csrc import attention_bf16 as A
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    lens = [1, 70, 200, 129, 64, 700]
    g = torch.Generator().manual_seed(hd + window)
    ks = [torch.randn(l, nkv, hd, generator=g) for l in lens]
    vs = [torch.randn(l, nkv, hd, generator=g) for l in lens]
    qs = [torch.randn(l, nh, hd, generator=g) * torch.linspace(0.05, 3.0, l)[:, None, None] for l in lens]
    pk, pv = Paged(lens, nkv, hd, torch.bfloat16, 3), Paged(lens, nkv, hd, torch.bfloat16, 3)
    pk.fill(ks, ks)
    pv.fill(vs, vs)
    k_d, v_d, tab = pk.dev()[0], pv.dev()[0], pk.dev()[2]
    rt = lambda a: a.bfloat16().double()
    full = [P.windowed_attention(rt(qs[b]), rt(ks[b]), rt(vs[b]), 0.3, window or None, True) for b in range(len(lens))]
    free = [P.windowed_attention(rt(qs[b]), rt(ks[b]), rt(vs[b]), 0.3, window or None, False) for b in range(len(lens))]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for new in ([1, 70, 67, 129, 5, 450], [1] * len(lens)):
        q = torch.cat([a[l - n:] for a, l, n in zip(qs, lens, new)]).reshape(sum(new), nh * hd).bfloat16().to(DEV)
        want = torch.cat([a[l - n:] for a, l, n in zip(full, lens, new)]).reshape(sum(new), -1).numpy()
        other = torch.cat([a[l - n:] for a, l, n in zip(free, lens, new)]).reshape(sum(new), -1).numpy()
        assert rel_err(other, want) > 0.1                                        # the sink matters here
        if max(new) > 1:
            got = [A.prefill(q, k_d, v_d, i32(np.concatenate([[0], np.cumsum(new)])), i32(lens), tab, len(lens), max(new), nh, 0.3,
                             window, status, kind=kind, sink=True)]
        else:
            got = [A.decode(q, k_d, v_d, i32(lens), tab, len(lens), max(lens), nh, 0.3, window, status, chunk_pages=c, sink=True)
                   for c in (1, 4)]
        assert status.item() == 0
        for o in got:
            assert rel_err(o.float().cpu().numpy(), want) < 8e-3


@pytest.mark.parametrize("nh,nkv,hd,hdv,window,sink", [(16, 1, 80, 64, 0, False), (3, 1, 80, 64, 70, False), (40, 1, 96, 64, 130, False),
                                                       (8, 2, 144, 128, 33, True), (5, 1, 64, 64, 64, False), (1, 1, 208, 192, 2, False)])
def test_attention_over_rows_that_hold_their_values(nh, nkv, hd, hdv, window, sink):
    """The bfloat16 kernel whose tile rows are (token, head) pairs of one key/value head: portions and single tokens over
    scrambled pages, few heads (several tokens in a tile), many (several tiles of heads), and single tokens of few
    sequences, whose pages are cut into runs that a second kernel merges."""
    from test_kernels_gpu import Paged
    from ithaca_b200.csrc import attention_latent as L
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    lens = [1, 70, 200, 129, 64, 700]
    g = torch.Generator().manual_seed(hd + window)
    ks = [torch.randn(l, nkv, hd, generator=g) for l in lens]
    qs = [torch.randn(l, nh, hd, generator=g) * torch.linspace(0.05, 1.5, l)[:, None, None] for l in lens]
    pk = Paged(lens, nkv, hd, torch.bfloat16, 3)
    pk.fill(ks, ks)
    k_d, tab = pk.dev()[0], pk.dev()[2]
    rt = lambda a: a.bfloat16().double()
    full = [P.windowed_attention(rt(qs[b]), rt(ks[b]), rt(ks[b])[:, :, :hdv], 0.2, window or None, sink) for b in range(len(lens))]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert L.supported(hd, hdv)
    for new in ([1, 70, 67, 129, 5, 450], [1] * len(lens)):
        q = torch.cat([a[l - n:] for a, l, n in zip(qs, lens, new)]).reshape(sum(new), nh * hd).bfloat16().to(DEV)
        want = torch.cat([a[l - n:] for a, l, n in zip(full, lens, new)]).reshape(sum(new), -1).numpy()
        ctx = SimpleNamespace(n_seqs=len(lens), max_new=max(new), kv_len_bound=max(lens), max_kv_len=max(lens), kv_lens=i32(lens),
                              cu_seqlens=i32(np.concatenate([[0], np.cumsum(new)])), host_n_new=new, host_kv_lens=lens)
        got = L.attend(q, k_d, ctx, tab, nh, 0.2, window, status, hdv, sink=sink)
        assert status.item() == 0
        assert rel_err(got.float().cpu().numpy(), want) < 8e-3, new[:2]
    # one long sequence alone: its pages are cut into many runs
    chunk, n = L.splits_for(1, 11)
    assert n > 1 and chunk * n >= 11
    b = len(lens) - 1
    ctx = SimpleNamespace(n_seqs=1, max_new=1, kv_len_bound=lens[b], max_kv_len=lens[b], kv_lens=i32([lens[b]]), cu_seqlens=i32([0, 1]),
                          host_n_new=[1], host_kv_lens=[lens[b]])
    got = L.attend(qs[b][-1:].reshape(1, nh * hd).bfloat16().to(DEV), k_d, ctx, tab[b:b + 1].contiguous(), nh, 0.2, window, status, hdv, sink=sink)
    assert status.item() == 0
    assert rel_err(got.float().cpu().numpy(), full[b][-1:].reshape(1, -1).numpy()) < 8e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_per_value_kernel(dtype):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    for H, hdv in ((5, 24), (3, 7)):
        T = 11
        att = torch.randn(T, H * hdv, generator=g).to(dtype)
        p = torch.randn(T, 3 + H * hdv + 2, generator=g)
        out = torch.zeros(T, H * hdv, dtype=dtype, device=DEV)
        ops.head_gate(att.to(DEV), p.to(DEV), 3, out, H, wide=True)
        want = att.double() * torch.sigmoid(p[:, 3:3 + H * hdv].double())
        assert rel_err(out.float().cpu().numpy(), want.numpy()) < (2e-6 if dtype == torch.float32 else 8e-3)
        same = att.clone().to(DEV)
        ops.head_gate(same, p.to(DEV), 3, same, H, wide=True)                   # in place
        assert torch.equal(same, out)


@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 24, 40, 3), (3, 3, 80, 16, 1), (1, 1, 16, 32, 4), (2, 1, 128, 64, 2), (2, 2, 64, 33, 4),
                                            (1, 1, 200, 8, 2)])
def test_gated_delta_rule_kernels(H, G, dk, dv, taps):
    """Convolution, unit vectors, steps, decays and the rule: three sequences in four steps (a prompt, a portion, two single
    tokens) against the plain recurrence over the whole sequences; states and rings start with another user's leftovers."""
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(dk + dv)
    C, pad = 2 * G * dk + H * dv, 3
    p = [torch.randn(l, pad + C + 2 * H, generator=g) for l in TOTAL]
    cw = torch.randn(C, taps, generator=g) * 0.6
    A_log, dt_bias = torch.randn(H, generator=g) * 0.5 - 0.5, torch.randn(H, generator=g) * 0.5 - 1.0
    state = torch.full((6, 2, H, dv, dk), 7.0, device=DEV)
    ring = torch.full((6, taps, C), 9.0, device=DEV) if taps > 1 else None
    got = [[] for _ in TOTAL]
    for lo, hi in STEPS:
        ctx = _ctx(lo, hi, [2, 0, 5])
        x = torch.cat([a[l:h] for a, l, h in zip(p, lo, hi)]).to(DEV)[:, pad:]
        u = ops.causal_conv(x[:, :C], cw.t().contiguous().to(DEV), None, ring, ctx, torch.float32, act=True)
        bg = ops.delta_prepare(u, 0, G * dk, x, C, C + H, A_log.to(DEV), dt_bias.to(DEV), G, dk, H, dk ** -0.5, 1e-6)
        o = ops.delta_rule(u, 0, G * dk, 2 * G * dk, bg, state, ctx, H, G, dk, dv)
        for i, part in enumerate(torch.split(o.cpu(), [h - l for l, h in zip(lo, hi)])):
            got[i].append(part)
    for i, l in enumerate(TOTAL):
        x = p[i][:, pad:].double()
        u = P.silu(P.short_convolution(x[:, :C], cw.double()))
        q, k, v = u[:, :G * dk].reshape(l, G, dk), u[:, G * dk:2 * G * dk].reshape(l, G, dk), u[:, 2 * G * dk:].reshape(l, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = P.sigmoid(x[:, C:C + H])
        a = torch.exp(-torch.exp(A_log.double()) * P.softplus(x[:, C + H:C + 2 * H] + dt_bias.double()))
        want = P.gated_delta_rule(q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1), v, beta, a)
        assert rel_err(torch.cat(got[i]).numpy(), want.reshape(l, -1).numpy()) < 5e-6, i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_gate_kernel(dtype):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(8)
    for H, dv in ((4, 40), (3, 7), (1, 300)):
        T = 13
        x, w, p = torch.randn(T, H * dv, generator=g) * 4, torch.randn(dv, generator=g), torch.randn(T, 5 + H * dv, generator=g)
        got = ops.head_norm_gate(x.to(DEV), w.to(DEV), 1e-5, p.to(DEV), 5, H, dtype, gate="silu")
        want = (P.rms_norm(x.double().view(T, H, dv), w, 1e-5).reshape(T, -1) * P.silu(p[:, 5:].double()))
        assert rel_err(got.float().cpu().numpy(), want.numpy()) < (3e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_per_head(dtype):
    """One launch, one product per head, operands and results as column ranges of wider rows; with 16-byte aligned heads
    (the last three) the 16-bit operands go through the tensor cores."""
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    for T, H, K, N, off, pad in ((70, 3, 16, 40, 2, 4), (5, 2, 40, 24, 2, 4), (130, 1, 33, 7, 2, 4), (200, 3, 32, 136, 8, 16),
                                 (5, 2, 128, 64, 0, 0), (300, 5, 72, 130, 8, 8)):
        x = torch.randn(T, H, K + pad, generator=g).to(dtype)
        w = torch.randn(H, N, K, generator=g).to(dtype)
        out = torch.zeros(T, H, N + 3, dtype=dtype, device=DEV)
        ops.gemm_heads(x.to(DEV)[:, :, off:off + K], w.to(DEV), out[:, :, 1:1 + N])
        want = torch.einsum("thk,hnk->thn", x[:, :, off:off + K].double(), w.double())
        assert rel_err(out[:, :, 1:1 + N].float().cpu().numpy(), want.numpy()) < (2e-6 if dtype == torch.float32 else 8e-3)
        assert float(out[:, :, 0].abs().max()) == 0.0 and float(out[:, :, 1 + N:].abs().max()) == 0.0


@pytest.mark.parametrize("act", ["relu2", "gelu_tanh"])
def test_activation_in_the_products_epilogue(act):
    """act(x W^T) in one kernel for few tokens (the skinny kernel) and many (tcgen05: whole tiles, slices of K, pairs of
    blocks), against the product in double with the activation applied to it."""
    from ithaca_b200.csrc import gemm_bf16
    g = torch.Generator().manual_seed(9)
    for M, N, K in ((3, 200, 64), (12, 136, 256), (40, 72, 1024), (300, 520, 128), (700, 264, 192), (129, 2048, 64)):
        x = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16()
        w = torch.randn(N, K, generator=g).bfloat16()
        got = gemm_bf16.gemm_act(x.to(DEV), w.to(DEV), act, torch.bfloat16)
        z = x.double() @ w.double().T
        want = torch.relu(z) ** 2 if act == "relu2" else 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        assert rel_err(got.float().cpu().numpy(), want.numpy()) < 8e-3, (M, N, K)


def _one_layer(kind, mixer, width=48, mlp=None):
    return {"architecture": "Mimadra", "vocab": 53, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


ONE_LAYER = {
    "attention": _one_layer("attention", _att(4, 2, 16, 24, 0.25, window=37, rot=(8, 100.0))),
    "attention, heads of their own": _one_layer("attention", _att(3, 3, 8, 8, 0.4, window=64, rot=(8, 10000.0)), mlp=_ff(32)),
    "delta": _one_layer("delta", _delta(4, 2, 16, 24, 4)),
    "delta, one tap": _one_layer("delta", _delta(2, 2, 48, 8, 1), mlp=_ff(40)),
    "latent": _one_layer("latent_attention", _lat(3, 16, 8, 24, 32, 0.2, 250.0, window=37)),
    "latent, a wide one": _one_layer("latent_attention", _lat(5, 16, 16, 24, 64, 0.2, 250.0, window=75)),
    "latent, no window": _one_layer("latent_attention", _lat(2, 24, 4, 8, 20, 0.3, 10000.0), mlp=_ff(24)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(ONE_LAYER))
def test_one_layer_models(tmp_path, which, dtype):
    """Each mixer as a model's only layer: a prompt with a neighbour, a portion, then single tokens."""
    from ithaca_b200 import Engine
    cfg = ONE_LAYER[which]
    t = make_tensors(cfg, 7)
    eng = Engine(_write(tmp_path, cfg, t, "one"), dtype=dtype, max_tokens=1024)
    reqs = {"a": random_ids(150, 53, 1), "b": random_ids(9, 53, 2)}
    got = run_schedule(eng, reqs, [[("a", 66), ("b", 3)], [("a", 70), ("b", 1)]] + [[("a", 1), ("b", 1)] for _ in range(5)]
                       + [[("a", 1)] for _ in range(9)])
    for r, ids in reqs.items():
        assert _close(got[r], _plain(cfg, t, ids), dtype), r


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_against_the_plain_model(models, name, dtype):
    from ithaca_b200 import Engine
    d, t = models[name]
    cfg = CONFIGS[name]
    V = cfg["vocab"]
    reqs = {"a": random_ids(141, V, 11), "b": random_ids(67, V, 12), "c": random_ids(1, V, 13), "d": random_ids(9, V, 14)}
    want = {r: _plain(cfg, t, ids) for r, ids in reqs.items()}
    eng = Engine(d, dtype=dtype, max_tokens=64 * 8)

    def portions(r, sizes):
        out, left, i = [], len(reqs[r]), 0
        while left:
            n = min(sizes[i % len(sizes)], left)
            out.append([(r, n)])
            left -= n
            i += 1
        return out
    schedules = {
        "whole": [[("a", 141)], [("b", 67)], [("c", 1)], [("d", 9)]],
        "token by token": [[("b", 1)] for _ in range(67)],
        "portions": portions("a", [2, 3, 7, 64, 65]),
        "pairs": portions("b", [2]),
        "prompt then decode": [[("a", 60)]] + [[("a", 1)] for _ in range(81)],
        "batch": [[("c", 1), ("a", 100), ("d", 5), ("b", 30)]] + [[("a", 1), ("d", 1), ("b", 1)] for _ in range(4)]
                 + [[("a", 1), ("b", 1)] for _ in range(33)] + [[("a", 1)] for _ in range(4)],
        "mixed portions": [[("a", 64), ("b", 1)], [("b", 64), ("a", 3)], [("a", 74), ("b", 2)]],
    }
    for label, sched in schedules.items():
        got = run_schedule(eng, reqs, sched)
        for r, lg in got.items():
            assert _close(lg, want[r], dtype), (label, r)
        eng.cache.table.check_consistent()
        assert eng.cache.table.n_slots_in_use() == 0


def test_float32_does_not_depend_on_the_cutting(models):
    """The recurrence runs token by token, attention reduces a query's keys in tiles that start at fixed positions, and every
    sum's order is fixed by sizes alone: in float32 two cuttings of the same tokens, alone or beside others, give the same bits."""
    from ithaca_b200 import Engine
    d, t = models["A"]
    reqs = {"a": random_ids(150, 101, 21), "b": random_ids(40, 101, 22)}
    eng = Engine(d, dtype="float32", max_tokens=2048)
    whole = run_schedule(eng, reqs, [[("a", 150)], [("b", 40)]])
    cut = run_schedule(eng, reqs, [[("a", 63), ("b", 2)], [("a", 2), ("b", 38)], [("a", 1)], [("a", 84)]])
    for r in reqs:
        assert np.array_equal(whole[r], cut[r]), r


def test_slots_pages_and_states_are_used_again(models):
    """A small cache: requests come and go, so slots, pages, states and rings are handed out again, also to shorter
    sequences whose first tokens must see nothing of what lay there before; windowed groups give pages back on the way."""
    from ithaca_b200 import Engine
    d, t = models["A"]
    eng = Engine(d, dtype="float32", max_tokens=64 * 6, max_slots=2)
    for round_ in range(4):
        reqs = {"x": random_ids(170 - 50 * round_, 101, 20 + round_), "y": random_ids(3 + round_, 101, 30 + round_)}
        got = run_schedule(eng, reqs, [[("x", len(reqs["x"]) - 2), ("y", 2)], [("x", 1), ("y", 1)], [("x", 1)]]
                           + [[("y", 1)] for _ in range(round_)])
        for r, ids in reqs.items():
            assert rel_err(got[r], _plain(CFG_A, t, ids)) < REL["float32"], (round_, r)
        eng.cache.table.check_consistent()


def test_a_reader_keeps_the_rows_its_wider_window_needs(models):
    """Layer 2 of configuration A reads layer 0's rows through a window of 100 while layer 0 itself looks back 70: the shared
    entry must keep pages for the wider of the two.  Decoding far past both windows gives pages back and still matches."""
    from ithaca_b200 import Engine
    d, t = models["A"]
    eng = Engine(d, dtype="float32", max_tokens=64 * 8)
    assert sorted(g.window for g in eng.cache.kv_groups if g.window is not None) == [33, 100]
    ids = random_ids(300, 101, 5)
    got = run_schedule(eng, {"a": ids}, [[("a", 130)]] + [[("a", 1)] for _ in range(170)])["a"]
    assert rel_err(got, _plain(CFG_A, t, ids)) < REL["float32"]
    held = max(pool.held() for pool in eng.cache.table.pools)
    assert held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    from ithaca_b200 import Engine
    d, t = models["A"]
    ids = random_ids(330, 101, 77)
    want = _plain(CFG_A, t, ids)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    got = run_schedule(eng, {"a": ids}, [[("a", 10)]] + [[("a", 1)] for _ in range(320)])["a"]
    assert _close(got, want, dtype)


# ------------------------------------------------------------------------------------------ one token decides
D = 32


def _needle_base(cfg):
    """Token 1 (the needle) and token 2 (the query) point along axis 0, every other token along an axis of its own; the
    needle carries a mark on axis 5."""
    t = make_tensors(cfg, 9)
    g = torch.Generator().manual_seed(1)
    emb = torch.randn(40, D, generator=g) * 0.05
    for i in range(3, 40):
        emb[i, 8 + i % 20] += 4.0
    emb[1] += torch.eye(D)[0] * 4 + torch.eye(D)[5] * 2
    emb[2] += torch.eye(D)[0] * 4 - torch.eye(D)[5] * 2
    t["embed"] = emb.bfloat16()
    for n in ("l0.norm1", "final.norm"):
        t[n] = torch.ones(D).bfloat16()
    t["l0.ls1"] = torch.full((D,), 3.0).bfloat16()                      # what the mixer adds outweighs the token's own embedding
    t["l0.mix.g"] = torch.zeros_like(t["l0.mix.g"])                     # a gate of one half everywhere
    return t


def _needle_attention(window):
    """k copies the input and q copies it with the mark's axis turned over, so the query's best match is the needle, ahead
    of itself and of hundreds of others; the value it fetches carries the needle's mark.  No rotation: distance plays no
    part in the score, only the window decides whether the needle is seen."""
    cfg = _one_layer("attention", _att(1, 1, D, D, 1.2, window=window), width=D)
    cfg["vocab"] = 40
    t = _needle_base(cfg)
    for r in "kvo":
        t[f"l0.mix.{r}"] = torch.eye(D).bfloat16()
    flip = torch.eye(D)
    flip[5, 5] = -1.0
    t["l0.mix.q"] = flip.bfloat16()
    t["l0.mix.q.norm"] = t["l0.mix.k.norm"] = torch.ones(D).bfloat16()
    return cfg, t


def _needle_latent(window):
    """The same through a latent: the down-projection copies the input into the latent (and nothing into the turning part),
    Wuk and Wuv copy the latent, q copies the input with the mark's axis turned over."""
    cfg = _one_layer("latent_attention", _lat(1, D, 2, D, D, 1.2, 100.0, window=window), width=D)
    cfg["vocab"] = 40
    t = _needle_base(cfg)
    flip = torch.eye(D)
    flip[5, 5] = -1.0
    t["l0.mix.q"] = torch.cat([flip, torch.zeros(2, D)]).bfloat16()
    t["l0.mix.dkv"] = torch.cat([torch.eye(D), torch.zeros(2, D)]).bfloat16()
    t["l0.mix.dkv.norm"] = torch.ones(D).bfloat16()
    t["l0.mix.uk"] = t["l0.mix.uv"] = t["l0.mix.o"] = torch.eye(D).bfloat16()
    return cfg, t


def _needle_delta():
    """A delta rule that hardly forgets (decays next to one): only the needle and the query have a key, along axis 0, and
    only the needle writes firmly, so what the query reads from the state is the needle's value, however long ago it was
    written."""
    cfg = _one_layer("delta", _delta(1, 1, D, D, 2), width=D)
    cfg["vocab"] = 40
    t = _needle_base(cfg)
    pick = torch.zeros(D, D)
    pick[0, 0] = 2.0                                                    # q and k: axis 0 only; silu(0) = 0 elsewhere
    t["l0.mix.q"] = t["l0.mix.k"] = pick.bfloat16()
    mark = torch.eye(D)
    mark[5, 5] = 3.0
    t["l0.mix.v"], t["l0.mix.o"] = mark.bfloat16(), torch.eye(D).bfloat16()
    last = torch.zeros(D, 2)
    last[:, 1] = 1.0                                                    # the convolution passes the current token through
    for r in "qkv":
        t[f"l0.mix.{r}.conv"] = last.bfloat16()
    t["l0.mix.g"] = torch.eye(D).bfloat16()
    t["l0.mix.g"][5, 5] = -1.0                                          # the query's gate is open where the needle's mark arrives
    t["l0.mix.norm"] = torch.ones(D).bfloat16()
    t["l0.mix.b"] = torch.zeros(1, D).bfloat16()
    t["l0.mix.b"][0, 5] = 2.0                                           # the mark decides the step: the needle writes firmly, the
    #                                                                     query hardly at all (a firm step would put its own value
    #                                                                     in the needle's place before reading)
    t["embed"][3:, 0] = 0.0                                             # the others' keys are exactly zero: they write nothing
    t["l0.mix.a"] = torch.zeros(1, D).bfloat16()
    t["l0.mix.dt_bias"] = torch.full((1,), -6.0).bfloat16()
    t["l0.mix.A_log"] = torch.zeros(1).bfloat16()
    return cfg, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("make", [lambda: _needle_attention(None), lambda: _needle_latent(None), _needle_delta],
                         ids=["attention", "latent", "delta"])
def test_the_one_early_token_that_matters(tmp_path, make, dtype):
    """The needle sits at the very start, at a page's last and first place and elsewhere far back; the query comes at the
    end of a prompt, is decoded alone after it, or follows a short portion; a batch neighbour runs beside it."""
    from ithaca_b200 import Engine
    cfg, t = make()
    d = _write(tmp_path, cfg, t, "needle")
    eng = Engine(d, dtype=dtype, max_tokens=4096)
    n = 400
    hay = [3 + (i * 7) % 37 for i in range(n)]
    tol = REL[dtype] if dtype == "float32" else 6e-2
    none = list(hay)
    none[n - 1] = 2
    base = _plain(cfg, t, none)[n - 1]
    for at in (0, 1, 63, 64, 127, 128, 300):
        ids = list(hay)
        ids[at], ids[n - 1] = 1, 2
        want = _plain(cfg, t, ids)[n - 1]
        assert rel_err(want, base) > 0.15, at                              # the test has teeth: without the needle, other logits
        for cut in (n, n - 1, n - 5, 65):
            s, other = eng.alloc_slot(), eng.alloc_slot()
            lg = eng.step([other, s], [hay[:7], ids[:cut]], "last")
            for x in ids[cut:]:
                lg = eng.step([s, other], [[x], [5]], "last")
            eng.free_slot(s)
            eng.free_slot(other)
            row = lg.cpu().numpy()[1 if cut == n else 0]
            assert rel_err(row, want) < tol, (at, cut)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 2, 37, 64, 65, 130])
@pytest.mark.parametrize("make", [_needle_attention, _needle_latent], ids=["attention", "latent"])
def test_a_windows_edge(tmp_path, make, window, dtype):
    """The needle stands exactly window - 1 positions before the query (the last place the window keeps) or window positions
    before it (the first it drops); the query ends a prompt, is decoded alone, or follows a short portion, at places where
    the window's edge falls on a page's border and inside a page.  Seen and unseen give logits far apart."""
    from ithaca_b200 import Engine
    cfg, t = make(window)
    d = _write(tmp_path, cfg, t, "edge")
    eng = Engine(d, dtype=dtype, max_tokens=2048)
    tol = REL[dtype] if dtype == "float32" else 6e-2
    for n in (window + 1, 150, 64 + window, 257):
        if n <= window:
            continue
        hay = [3 + (i * 7) % 37 for i in range(n)]
        rows = {}
        for back in (window - 1, window):
            ids = list(hay)
            ids[n - 1] = 2
            if back > 0:
                ids[n - 1 - back] = 1                                     # back = 0: the query is its own only key
            want = _plain(cfg, t, ids)[n - 1]
            rows[back] = want
            for cut in (n, n - 1, max(1, n - 3)):
                s = eng.alloc_slot()
                lg = eng.step([s], [ids[:cut]], "last")
                for x in ids[cut:]:
                    lg = eng.step([s], [[x]], "last")
                eng.free_slot(s)
                assert rel_err(lg.cpu().numpy()[0], want) < tol, (n, back, cut)
        if window > 1:
            assert rel_err(rows[window - 1], rows[window]) > 0.15, n       # the edge has teeth
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_the_weight_when_nothing_matches(tmp_path, dtype):
    """Queries that match no key well (scores far below zero): with the sink the mixer adds next to nothing, without it the
    softmax would still hand out all its weight.  The first tokens of a sequence (one key, two keys) are such queries."""
    from ithaca_b200 import Engine
    cfg, t = _needle_attention(None)
    t["l0.mix.q"] = (-t["l0.mix.k"].float()).bfloat16()                  # every query points away from every key like it
    d = _write(tmp_path, cfg, t, "sink")
    eng = Engine(d, dtype=dtype, max_tokens=512)
    ids = [1 + (i * i // 3) % 2 for i in range(70)]                          # two tokens whose keys lie close to each other
    want = _plain(cfg, t, ids)
    got = run_schedule(eng, {"a": ids}, [[("a", 1)], [("a", 1)], [("a", 2)], [("a", 64)], [("a", 1)], [("a", 1)]])["a"]
    assert rel_err(got, want) < (REL[dtype] if dtype == "float32" else 6e-2)
    x = t["embed"].double()[torch.tensor(ids)]
    alone = P.rms_norm(x, t["final.norm"], 1e-5) @ t["head"].double().T
    alone = 20.0 * torch.tanh(alone / 20.0)
    assert rel_err(want, alone.numpy()) < 0.1                             # the mixer added next to nothing


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """More prompts than slots, unequal lengths, the generation loop's own batching (and its graph-replayed decode
    steps, which launch a step ahead and may drop it: the states are kept by parity so that this changes nothing)."""
    from ithaca_b200 import Engine
    d, t = models[name]
    V = CONFIGS[name]["vocab"]
    prompts = [random_ids(n, V, 60 + n) for n in (1, 6, 70, 20)]
    eng = Engine(d, dtype="float32", max_tokens=64 * 12, max_slots=3, graphs=graphs)
    assert (eng._decoder is not None) == graphs                            # every part of the design may be replayed
    got = eng.generate(prompts, max_tokens=12, temp=0.0, rep_pen=1.0, stop_token_ids=[])

    def check(p, g):
        lgs = P.forward(CONFIGS[name], t, list(p) + g[:-1])
        for i, tok in enumerate(g):
            lg = lgs[len(p) - 1 + i]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg.abs().max()):
                assert tok == int(lg.argmax()), (len(p), i)
    for p, g in zip(prompts, got):
        assert len(g) == 12
        check(p, g)
    assert eng.cache.table.n_slots_in_use() == 0
    # requests that end at different times: the step launched ahead is dropped when the batch changes
    got = eng.generate(prompts[:3], max_tokens=9, temp=0.0, rep_pen=1.0, stop_token_ids=[got[0][4], got[2][6]])
    for p, g in zip(prompts, got):
        check(p, g)


# ------------------------------------------------------------------------------------------ the programs
def test_trace_replay_and_command_line(models, tmp_path):
    import subprocess
    import sys
    from helpers import ROOT
    d, t = models["A"]
    V = 101
    reqs = {"p": random_ids(70, V, 90), "q": random_ids(3, V, 91), "r": random_ids(130, V, 92)}
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": reqs["p"][:66], "want": [0, 65]}, {"id": "q", "tokens": reqs["q"][:1], "want": []},
                                     {"id": "r", "tokens": reqs["r"][:126], "want": [125]}], "end": []}]
    for i in range(4):
        ent = [{"id": "p", "tokens": [reqs["p"][66 + i]], "want": [0]}, {"id": "r", "tokens": [reqs["r"][126 + i]], "want": [0]}]
        if i < 2:
            ent.insert(1, {"id": "q", "tokens": [reqs["q"][1 + i]], "want": [0] if i == 1 else []})
        steps.append({"step": 1 + i, "entries": ent, "end": (["q"] if i == 1 else []) + (["p", "r"] if i == 3 else [])})
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "210"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                           timeout=900)
        assert p.returncode == 0, p.stderr[-3000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
        want = {r: _plain(CFG_A, t, ids) for r, ids in reqs.items()}
        tol = REL[dtype] * (1 if dtype == "float32" else 2)
        got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V)
        assert rel_err(got0, np.stack([want["p"][0], want["p"][65], want["r"][125]])) < tol
        got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(3, V)
        assert rel_err(got2, np.stack([want["p"][67], want["q"][2], want["r"][127]])) < tol
        got4 = np.fromfile(out / "4.f32", dtype="<f4").reshape(2, V)
        assert rel_err(got4, np.stack([want["p"][69], want["r"][129]])) < tol

    cli = [sys.executable, os.path.join(ROOT, "bin", "ithaca"), "--model", d, "--dtype", "float32"]
    p = subprocess.run(cli + ["--describe"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and p.stdout.count("prenorm") == 6 and p.stdout.count("gated_delta") == 2 \
        and p.stdout.count("latent_attention") == 2 and p.stdout.count("read only") == 1, p.stderr[-2000:]
    prompt = random_ids(11, V, 93)
    p = subprocess.run(cli + ["--prompt", ",".join(map(str, prompt)), "-n", "5", "--rep-pen", "1.0", "--stop-ids", ""],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    from ithaca_b200 import Engine
    eng = Engine(d, dtype="float32", max_tokens=512)
    assert [int(x) for x in p.stdout.strip().split(",")] == eng.generate([prompt], max_tokens=5, temp=0.0, rep_pen=1.0, stop_token_ids=[])[0]
