"""Attention over bfloat16 key rows that carry their own values (a latent that is key and value at once): one compiled
module per (row size, value size).

``attention_latent.cu`` makes the query heads of a key/value group the rows of its tensor-core tile, so a cached row is
read once for all of them.  The module for the sizes a model has is compiled the first time that model runs a step.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import build
from . import ops
from .ops import KernelError, _check, _ptr, _stream, sm_count

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_modules: Dict[Tuple[int, int], ctypes.CDLL] = {}

ROWS = 32                     # (token, head) rows of a block
SMEM_LIMIT = 227 * 1024


def supported(row_size: int, value_size: int) -> bool:
    """Rows in multiples of 16, values in multiples of 64 (four column groups of whole 16-wide tiles), and two pages,
    the queries and the weights must fit into a block's shared memory."""
    if row_size % 16 or value_size % 64 or not 64 <= value_size <= row_size:
        return False
    ld = row_size + 8
    return (ROWS * ld + 2 * 64 * ld + ROWS * 72) * 2 + 512 <= SMEM_LIMIT


def module(row_size: int, value_size: int) -> ctypes.CDLL:
    key = (row_size, value_size)
    m = _modules.get(key)
    if m is None:
        m = build.load_library(f"ithaca_attn_latent_{row_size}_{value_size}", ["attention_latent.cu"],
                               defines=[f"IK_HD={row_size}", f"IK_HDV={value_size}"])
        m.ik_attn_latent.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _i, _i, _vp, _vp]
        m.ik_attn_latent.restype = _i
        if m.ik_attn_latent_rows() != ROWS:
            raise KernelError("the latent attention module was compiled for another tile")
        _modules[key] = m
    return ops.timed(m)


def splits_for(n_blocks: int, pages: int, n_sm: Optional[int] = None) -> Tuple[int, int]:
    """(pages per split, splits) for blocks that would each walk ``pages`` pages: about two blocks per SM when the
    step has fewer, in runs of at least two pages."""
    n_sm = n_sm if n_sm is not None else sm_count()
    want = max(1, (2 * n_sm) // max(n_blocks, 1))
    chunk = max(2, -(-pages // want))
    if chunk >= pages:
        return pages, 1
    return chunk, -(-pages // chunk)


def attend(q: torch.Tensor, k_pages: torch.Tensor, ctx, table: torch.Tensor, n_heads: int, scale: float, window: int,
           status: Optional[torch.Tensor], value_size: int, sink: bool = False) -> Optional[torch.Tensor]:
    """q [T, n_heads * row size] against the rows of ``k_pages`` [pages, kv heads, 64, row size]; a row's leading
    ``value_size`` columns are its value.  Returns [T, n_heads * value_size], or None when the kernel does not take
    these sizes or types (the caller then uses the CUDA-core kernel)."""
    n_pages, nkv, page_size, hd = k_pages.shape
    if k_pages.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or page_size != 64 or not supported(hd, value_size):
        return None
    if n_heads % nkv or q.shape[1] != n_heads * hd:
        raise KernelError("latent attention: q has the wrong shape")
    T, B = q.shape[0], ctx.n_seqs
    group = n_heads // nkv
    hpb = min(group, ROWS)
    tpb = ROWS // hpb
    # pages a block's rows can see, from the bound (a captured graph is replayed for other lengths)
    bound = max(ctx.kv_len_bound, ctx.max_kv_len, 1)
    reach = min(bound, window + tpb) if window else bound
    pages = -(-reach // page_size) + (1 if window else 0)
    chunk, n_splits = pages, 1
    if ctx.max_new == 1:
        chunk, n_splits = splits_for(B * nkv * -(-group // hpb), pages)
    out = torch.empty((T, n_heads * value_size), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T * n_heads, n_splits, value_size), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * n_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    if ops.profiling():
        pairs = 0
        for n, end in zip(ctx.host_n_new, ctx.host_kv_lens):
            for p in range(end - n, end):
                pairs += min(p + 1, window) if window else p + 1
        keys = sum(min(e, window + n) if window else e for n, e in zip(ctx.host_n_new, ctx.host_kv_lens))
        ops._work(f"attention latent {T}x{n_heads}", ops._nbytes(q, out) + keys * nkv * hd * 2, 2 * pairs * n_heads * (hd + value_size))
    m = module(hd, value_size)
    _check(m.ik_attn_latent(_ptr(q), _ptr(k_pages), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(ctx.cu_seqlens),
                            _ptr(ctx.kv_lens), _ptr(table), table.stride(0), T, B, ctx.max_new, n_heads, nkv, scale,
                            int(window or 0), 1 if sink else 0, page_size, n_pages, chunk, n_splits, _ptr(status), _stream()),
           "attention latent", kernels=2 if n_splits > 1 else 1)
    return out
