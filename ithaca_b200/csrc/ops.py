"""Python side of the kernel library: argument checks, pointers, the current stream.

Every function launches on torch's current CUDA stream and allocates nothing but its
declared outputs.  A non-zero status from the library raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_vp, _i, _f, _u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


_launches = 0


def launch_count() -> int:
    """Kernel-library calls made so far in this process (each is one or two kernel launches)."""
    return _launches


def _check(status: int, what: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: bad argument")
    if status == -2:
        raise KernelError(f"{what}: these sizes are not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {status} at launch")


_SIGNATURES = {
    "ik_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp, _vp],
    "ik_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "ik_swiglu": [_vp, _vp, _i, _i, _i, _i, _vp],
    "ik_fill_random": [_vp, _i, _u64, _u64, _f, _f, _vp],
    "ik_device_sm_count": [],
    "ik_copy": [_vp, _vp, _u64, _vp],
    "ik_rope_append": [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_gemm_bf16_mma_batched": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, _vp],
    "ik_gemm_bf16_mma": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f, _vp],
    "ik_gemm_tcgen05": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f, _i, _vp, _vp],
    "ik_gemm_tcgen05_tile": [_i],
    "ik_gemm_tcgen05_tile_width": [_i, _i],
    "ik_gemm_tcgen05_stream_k_bytes": [],
    "ik_rope_table": [_vp, _vp, _vp, _i, _i, _vp],
    "ik_gemm_qkv_rope_mma": [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_gemm_qkv_rope_tcgen05": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "ik_attention_simt": [_vp, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i, _vp, _i, _i, _vp, _vp],
    "ik_gemm_simt_batched": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _u64, _u64, _u64, _vp],
    "ik_scale_add_norm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "ik_plain_act": [_vp, _vp, _i, _u64, _i, _vp],
    "ik_delta_prepare": [_vp, _i, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp],
    "ik_delta_rule": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_head_norm_gate": [_vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _f, _i, _i, _vp],
    "ik_latent_prepare": [_vp, _i, _i, _i, _vp, _f, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                          _vp, _vp],
    "ik_layernorm": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _f, _i, _i, _f, _vp],
    "ik_add": [_vp, _vp, _u64, _vp],
    "ik_conv_rope_append": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i,
                            _i, _i, _i, _i, _i, _vp, _vp],
    "ik_moe_tile_rows": [],
    "ik_moe_route": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_moe_router": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_moe_sort": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ik_moe_gemm": [_i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _vp],
    "ik_moe_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ik_moe_sort_padded": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_moe_gather": [_vp, _vp, _vp, _i, _i, _vp],
    "ik_moe_gather_scaled": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "ik_gemm_tcgen05_grouped": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "ik_argmax": [_vp, _i, _vp, _i, _i, _vp, _vp],
    "ik_argmax_scratch_bytes": [],
    "ik_selftest_wait_expires": [_vp, _vp, _vp, _u64, _vp],
    "ik_gemm_tcgen05_issue_rate": [_i, _i, _i, _vp, _vp, _vp],
    "ik_gemm_tcgen05_take_wait_record": [_vp],
    "ik_sample": [_vp, _i, _vp, _vp, _i, _i, _f, _i, _f, _f, _vp, _i, _u64, _vp, _vp, _vp],
    "ik_rmsnorm_add": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _f, _vp],
    "ik_cast": [_vp, _i, _vp, _i, _i, _i, _i, _vp],
    "ik_scale_softcap": [_vp, _u64, _f, _f, _vp],
    "ik_glu_act": [_vp, _vp, _i, _i, _i, _i, _f, _f, _f, _vp],
    "ik_causal_conv": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_selective_scan": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "ik_decay_attention": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ik_norm_rope_append": [_vp, _i, _i, _i, _i, _vp, _vp, _f, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _f, _i, _i, _i, _i,
                            _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp],
    "ik_head_gate": [_vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ik_gated_rmsnorm": [_vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _f, _f, _vp],
    "ik_hyper_start": [_vp, _vp, _i, _i, _i, _vp],
    "ik_add_rows": [_vp, _vp, _i, _i, _vp],
    "ik_hyper_read": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp],
    "ik_hyper_write": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp],
    "ik_branch_norm_sum": [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _f, _i, _vp],
    "ik_rmsnorm_range": [_vp, _i, _vp, _vp, _i, _i, _i, _f, _vp],
    "ik_decay_rows": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ik_token_shift": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _i, _i, _i, _i, _i, _vp],
    "ik_row_decay": [_i, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
}

_lib = None
_status = {}


# ---------------------------------------------------------------------------------------------
# Per-kernel timing.  The reference times each operation of a forward pass when ITHACA_PROF is set
# (src/model.cpp:1261-1307, src/cuda_tier.cpp:514-527).  Here, while a ``Profile`` is active, every call
# into the kernel library is bracketed by CUDA events; the wrappers below say beforehand how many bytes the call has
# to move and how many floating-point operations it has to do, so that a table can hold each call against the
# device's peaks.  The events keep kernels from overlapping (no early launch), and nothing may be captured into
# a graph meanwhile: it is a tool for looking at a step, not the way a step runs.
class Profile:
    def __init__(self):
        self.records = []            # (label, start event, end event, bytes, flops)

    def __enter__(self):
        global _profile
        if _profile is not None:
            raise KernelError("a kernel profile is already being taken")
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile, _pending
        _profile, _pending = None, None
        return False

    def rows(self):
        """Per label, in order of first appearance: calls, microseconds, bytes, flops."""
        torch.cuda.synchronize()
        out = {}
        for label, e0, e1, nbytes, flops in self.records:
            r = out.setdefault(label, {"kernel": label, "calls": 0, "us": 0.0, "bytes": 0, "flops": 0})
            r["calls"] += 1
            r["us"] += e0.elapsed_time(e1) * 1e3
            r["bytes"] += nbytes
            r["flops"] += flops
        return list(out.values())


_profile: Optional[Profile] = None
_pending = None                      # (label, bytes, flops) of the library call that comes next


def profiling() -> bool:
    return _profile is not None


def _work(label: str, nbytes: int = 0, flops: int = 0) -> None:
    global _pending
    if _profile is not None:
        _pending = (label, int(nbytes), int(flops))


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


class _TimedLibrary:
    """Stands in for a loaded library while a profile is taken."""

    def __init__(self, library):
        self._library = library

    def __getattr__(self, name):
        fn = getattr(self._library, name)
        if _profile is None or not name.startswith("ik_") or fn.argtypes is None or not fn.argtypes or fn.argtypes[-1] is not _vp:
            return fn                                        # not a launch (no stream argument)

        def call(*args):
            global _pending
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            st = fn(*args)
            e1.record()
            label, nbytes, flops = _pending or (name[3:], 0, 0)
            _pending = None
            _profile.records.append((label, e0, e1, nbytes, flops))
            return st
        return call


def timed(library):
    return _TimedLibrary(library) if _profile is not None else library


def device_status(device) -> torch.Tensor:
    """The int32 status word kernels set when they meet something they refuse to do (an index
    out of range, a wait that ran out); one per device, shared by every runtime on it."""
    key = str(torch.device(device))
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def lib():
    """The loaded kernel library; built on first use.  Raises if that fails."""
    global _lib
    if _lib is None:
        l = build.core()
        for name, sig in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = sig
            fn.restype = _i
        _lib = l
    return timed(_lib)


# ---------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, status: Optional[torch.Tensor] = None,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, d) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=ids.device)
    _work(f"embed {T}x{d}", T * d * (table.element_size() + 4))
    _check(lib().ik_embed(_ptr(ids), _ptr(table), _code(table), _ptr(out), T, d, V, scale, _ptr(status), _stream()),
           "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_in: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    d = x.shape[-1]
    if weight.numel() != d:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} elements, rows have {d}")
    rows = x.numel() // d if rows_in is None else rows_in.numel()
    if rows_in is not None:
        _need(rows_in, "rows_in", torch.int32)
    if out is None:
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
    _work(f"rmsnorm {rows}x{d}", rows * d * (4 + out.element_size()) + d * 4)
    _check(lib().ik_rmsnorm(_ptr(x), _ptr(rows_in), _ptr(weight), _ptr(out), _code(out), rows, d, eps, _stream()),
           "rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
           interleaved: bool = False) -> torch.Tensor:
    """``interleaved``: gate j and up j sit in columns 2j and 2j + 1 instead of j and ff + j."""
    _need(gate_up, "gate_up", torch.float32)
    T, ff2 = gate_up.shape
    if ff2 % 2:
        raise KernelError("swiglu: the input needs an even number of columns (gate then up)")
    if out is None:
        out = torch.empty((T, ff2 // 2), dtype=out_dtype, device=gate_up.device)
    _work(f"swiglu {T}x{ff2 // 2}", _nbytes(gate_up, out))
    _check(lib().ik_swiglu(_ptr(gate_up), _ptr(out), _code(out), T, ff2 // 2, 1 if interleaved else 0, _stream()), "swiglu")
    return out


def fill_random(out: torch.Tensor, key: int, scale: float, offset: float) -> torch.Tensor:
    """Fills ``out`` with offset + scale * (a centred sum of eight 16-bit hash fields) per flat index; the values are
    the ones ``weights.random_init.hashed_normal`` gives on the host for the same key."""
    _need(out, "out")
    _check(lib().ik_fill_random(_ptr(out), _code(out), out.numel(), key & 0xFFFFFFFFFFFFFFFF, scale, offset, _stream()),
           "fill_random")
    return out


def copy(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """dst = src with this library's streaming copy kernel (sizes a multiple of 16 bytes)."""
    _need(src, "src")
    _need(dst, "dst")
    n = src.numel() * src.element_size()
    if n != dst.numel() * dst.element_size():
        raise KernelError("copy: source and destination differ in size")
    _work(f"copy {n >> 20} MiB", 2 * n)
    _check(lib().ik_copy(_ptr(src), _ptr(dst), n, _stream()), "copy")
    return dst


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                inv_freq: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                pairing: int, write_cache: bool, status: Optional[torch.Tensor]) -> None:
    """k_pages / v_pages: [n_pages, n_kv_heads, page_size, head_dim] of one layer."""
    _need(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages")
    _need(table, "table", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope_append: qkv has the wrong width")
    n_pages, nkv, page_size, hd = k_pages.shape
    if nkv != n_kv_heads or hd != head_dim or v_pages.shape != k_pages.shape or v_pages.dtype != k_pages.dtype:
        raise KernelError("rope_append: the pages do not match the head sizes")
    _work(f"rope_append {T}", _nbytes(qkv, q_out) + 2 * T * n_kv_heads * head_dim * k_pages.element_size())
    _check(lib().ik_rope_append(_ptr(qkv), _ptr(q_out), _code(q_out), _ptr(k_pages), _ptr(v_pages), _code(k_pages),
                                _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), _ptr(inv_freq), T,
                                n_heads, n_kv_heads, head_dim, rotary_dim, pairing, page_size, n_pages,
                                1 if write_cache else 0, _ptr(status), _stream()), "rope_append")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
              accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (+)= x[M, K] @ w[N, K]^T on the CUDA cores, float accumulation in ascending k."""
    _need(x, "x", contiguous=False)
    _need(w, "w", contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    _work(f"gemm_simt {M}x{N}x{K}", M * K * x.element_size() + N * K * w.element_size() + M * N * out.element_size(), 2 * M * N * K)
    _check(lib().ik_gemm_simt(_ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), M, N, K, x.stride(0),
                              w.stride(0), out.stride(0), 1 if accumulate else 0, _stream()), "gemm_simt")
    return out


def _act_code(act: Optional[str], joins: bool = False) -> int:
    """What a product's epilogue is told when it applies an ungated activation to every result (``PLAIN_ACTS``): 16 + its
    number; 0 = none.  Not together with a gate/up join."""
    if act is None:
        return 0
    if joins:
        raise KernelError("gemm: an activation on every result and a gate/up join exclude each other")
    return 16 + PLAIN_ACTS[act]


def gemm_bf16_mma(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                  accumulate: bool = False, kind: int = 0, swiglu: bool = False, glu=None, act: Optional[str] = None) -> Optional[torch.Tensor]:
    """bfloat16 operands, float accumulation on the warp-level tensor-core path.  ``kind``: 0 = by
    M, 1 = the skinny (decode) kernel, 2 = the tiled kernel.  Returns None when the kernels
    do not take these sizes (K not a multiple of 8, unaligned rows).  ``glu`` = (alpha, limit, shift) with ``swiglu``: the
    epilogue joins gate and up as gate * sigmoid(alpha gate) * (up + shift), both limited, instead of silu(gate) * up.

    ``w`` is a weight: the skinny kernel, launched early, reads its first rows before it waits for the
    kernel before it in the stream, so ``w`` must not be what that kernel writes (``x`` and ``out`` may be)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    _work(f"gemm_skinny{' +swiglu' if swiglu else ''}{' +' + act if act else ''} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
    ga, gl, gs = glu if glu is not None else (1.0, 0.0, 0.0)
    join = (2 if glu is not None else 1) if swiglu else _act_code(act, swiglu)
    st = lib().ik_gemm_bf16_mma(_ptr(x), _ptr(w), _ptr(out), _code(out), M, N, K, x.stride(0), w.stride(0),
                                out.stride(0), 1 if accumulate else 0, kind, join, ga, gl, gs,
                                _stream())
    if st == -2:
        return None
    _check(st, "gemm_bf16_mma")
    return out


_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(lib().ik_device_sm_count())
    return n


_stream_k_scratch = {}


def stream_k_scratch(device) -> torch.Tensor:
    """Scratch of the stream-K product (pieces of tiles and their flags): one per device, zeroed once; the
    kernels leave the flags zero.  Launches that use it must follow one another in one stream."""
    key = str(torch.device(device))
    t = _stream_k_scratch.get(key)
    if t is None:
        t = torch.zeros(lib().ik_gemm_tcgen05_stream_k_bytes() // 4, dtype=torch.float32, device=device)
        _stream_k_scratch[key] = t
    return t


def tcgen05_cluster_fits(M: int, N: int, K: int, n_cl: int) -> bool:
    """Whether the cluster mode of the tcgen05 product takes this shape with ``n_cl`` blocks per tile."""
    tile_m = lib().ik_gemm_tcgen05_tile(M)
    tiles = -(-N // 128) * -(-M // tile_m)
    steps = -(-K // 64)
    most = 4 if tile_m <= 64 else 2 if tile_m <= 128 else 1
    return 2 <= n_cl <= most and tiles * n_cl <= sm_count() and (n_cl - 1) * -(-steps // n_cl) < steps


def tcgen05_splits(M: int, N: int, K: int) -> int:
    """How the tcgen05 product shares out its work: 1 = whole tiles dealt round robin; n > 1 = n slices
    of K and a second kernel that adds them; 0 = stream-K (equal shares of all K steps of all tiles);
    -n = clusters of n blocks per tile, each a slice of K, summed in shared memory (no scratch, one kernel).
    Measured on B200 with 2048 x 2048 .. 28672 x 4096 weights (``bench.py --only products --tokens ...``): with
    fewer tiles than half the SMs, K is sliced: by clusters of 2 or 4 where that busies at least half the SMs (clusters
    of 3 measured far slower), else by a second kernel; stream-K wins when whole tiles would leave more than a
    tenth of the SMs' time unused and there is one token tile of at most 128 tokens (bandwidth-bound); beyond that
    whole tiles win."""
    N_SM = sm_count()
    tile_m = lib().ik_gemm_tcgen05_tile(M)
    tiles_m = -(-M // lib().ik_gemm_tcgen05_tile_width(M, N))
    tiles = -(-N // 128) * tiles_m
    steps = -(-K // 64)
    if 2 * tiles <= N_SM:
        want = max(1, min(N_SM // tiles, steps // 4))
        most = 4 if tile_m <= 64 else 2 if tile_m <= 128 else 1
        n_cl = 4 if want >= 4 and most >= 4 else 2 if want >= 2 and most >= 2 else 0
        if n_cl and 2 * tiles * n_cl >= N_SM and tcgen05_cluster_fits(M, N, K, n_cl):
            return -n_cl
        return want
    rounds = -(-tiles // N_SM)
    if tiles_m == 1 and tile_m <= 128 and tiles / (rounds * N_SM) < 0.9 and tiles * steps >= 8:
        return 0
    return 1


_pairs_lib = None
PAIRS = os.environ.get("IK_PAIRS", "1") != "0"


def pairs_lib():
    """The pair mode of the tcgen05 product (two blocks share one copy of a token tile: less traffic from L2 at
    prefill), a library of its own; None where its source is not there or ``IK_PAIRS=0`` says not to use it."""
    global _pairs_lib
    if _pairs_lib is None:
        if not PAIRS or not build.pairs_available():
            _pairs_lib = False
        else:
            l = build.pairs()
            l.ik_gemm_tcgen05_pairs.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f, _vp, _vp]
            l.ik_gemm_tcgen05_pairs.restype = _i
            l.ik_gemm_qkv_rope_tcgen05_pairs.argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]
            l.ik_gemm_qkv_rope_tcgen05_pairs.restype = _i
            _pairs_lib = l
    return timed(_pairs_lib) if _pairs_lib else None


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                 accumulate: bool = False, splits: Optional[int] = None,
                 status: Optional[torch.Tensor] = None, swiglu: bool = False, pairs: Optional[bool] = None,
                 glu=None, act: Optional[str] = None) -> Optional[torch.Tensor]:
    """bfloat16 operands on the tcgen05 tensor cores (TMA-fed, accumulators in TMEM).  Returns None
    when the kernel does not take these sizes (K not a multiple of 8, unaligned rows).

    ``w`` is a weight: launched early, the kernel asks for its first tiles of ``w`` before it waits for the
    kernel before it in the stream, so ``w`` must not be what that kernel writes (``x`` and ``out`` may be)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match or rows are not contiguous")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return None
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output to add to")
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    _need(out, "out", contiguous=False)
    if out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError("gemm: the output has the wrong shape")
    if splits is None:
        splits = tcgen05_splits(M, N, K)
    # ``glu`` = (alpha, limit, shift): the gate with parameters; ``act``: an ungated activation on every result
    join = (2 if glu is not None else 1) if swiglu else _act_code(act, swiglu)
    tag = (' +swiglu' if swiglu else '') + (' +' + act if act else '')
    ga, gl, gs = glu if glu is not None else (1.0, 0.0, 0.0)
    if splits == 1 and M > 256 and pairs is not False:
        pl = pairs_lib()
        if pl is None and pairs:
            raise KernelError("gemm_tcgen05: the pair mode was asked for but its library is not there")
        if pl is not None:
            _work(f"gemm_tcgen05 pairs{tag} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
            st = pl.ik_gemm_tcgen05_pairs(_ptr(x), _ptr(w), _ptr(out), _code(out), M, N, K, x.stride(0), w.stride(0),
                                          out.stride(0), 1 if accumulate else 0, join, ga, gl, gs, _ptr(status), _stream())
            if st != -2:
                _check(st, "gemm_tcgen05 (pairs)")
                return out
    partial = (stream_k_scratch(x.device) if splits == 0 else
               torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None)
    _work(f"gemm_tcgen05{tag} {M}x{N}x{K}", 2 * (M * K + N * K) + M * n_out * out.element_size(), 2 * M * N * K)
    st = lib().ik_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), _code(out), _ptr(partial), M, N, K, x.stride(0),
                               w.stride(0), out.stride(0), 1 if accumulate else 0, join, ga, gl, gs, splits, _ptr(status),
                               _stream())
    if st == -2:
        return None
    _check(st, "gemm_tcgen05", kernels=2 if splits > 1 else 1)
    return out


class RopeStore(ctypes.Structure):
    """Mirror of IkRopeStore (rope_store.cuh): where the fused q/k/v product puts its results."""
    _fields_ = [("q_out", _vp), ("k_pages", _vp), ("v_pages", _vp), ("cos_sin", _vp), ("token_seq", _vp),
                ("token_pos", _vp), ("table", _vp), ("status", _vp), ("table_stride", _i), ("nh", _i), ("nkv", _i),
                ("hd", _i), ("page_size", _i), ("n_pages", _i), ("write_cache", _i)]


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[T, half, 2] float: cos and sin of float(pos) * inv_freq, for the fused q/k/v epilogue."""
    _need(token_pos, "token_pos", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    T, half = token_pos.numel(), inv_freq.numel()
    out = torch.empty((T, half, 2), dtype=torch.float32, device=token_pos.device)
    _work(f"rope_table {T}", T * half * 8)
    _check(lib().ik_rope_table(_ptr(token_pos), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_table")
    return out


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                  cos_sin: torch.Tensor, token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                  n_heads: int, n_kv_heads: int, head_dim: int, write_cache: bool, status: Optional[torch.Tensor],
                  skinny_max: int = 16, splits: Optional[int] = None) -> bool:
    """q, k, v = x W^T with rotary pairs in adjacent rows of W; rotated q to ``q_out``, rotated k and v into
    the pages.  Returns False when the kernels do not take these sizes (the caller then runs the steps apart)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16, contiguous=False)
    _need(q_out, "q_out", torch.bfloat16)
    _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32)
    _need(table, "table", torch.int32)
    M, K = x.shape
    N = w.shape[0]
    n_pages, nkv, page_size, hd = k_pages.shape
    if (N != (n_heads + 2 * n_kv_heads) * head_dim or nkv != n_kv_heads or hd != head_dim or head_dim % 2
            or cos_sin.shape != (M, head_dim // 2, 2) or q_out.shape != (M, n_heads * head_dim)):
        raise KernelError("gemm_qkv_rope: the sizes do not fit together")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or x.stride(1) != 1 \
            or w.stride(1) != 1:
        return False
    rs = RopeStore(_ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(cos_sin), _ptr(token_seq), _ptr(token_pos),
                   _ptr(table), _ptr(status), table.stride(0), n_heads, n_kv_heads, head_dim, page_size, n_pages,
                   1 if write_cache else 0)
    _work(f"gemm_{'skinny' if M <= skinny_max else 'tcgen05'} +rope+cache {M}x{N}x{K}", 2 * (M * K + N * K + M * N), 2 * M * N * K)
    if M <= skinny_max:
        st = lib().ik_gemm_qkv_rope_mma(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), ctypes.byref(rs), _stream())
        kernels = 1
    else:
        if splits is None:
            splits = tcgen05_splits(M, N, K)
        pl = pairs_lib() if splits == 1 and M > 256 else None
        if pl is not None:
            st = pl.ik_gemm_qkv_rope_tcgen05_pairs(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), _ptr(status),
                                                   ctypes.byref(rs), _stream())
            if st != -2:
                _check(st, "gemm_qkv_rope (pairs)")
                return True
        partial = (stream_k_scratch(x.device) if splits == 0 else
                   torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None)
        st = lib().ik_gemm_qkv_rope_tcgen05(_ptr(x), _ptr(w), _ptr(partial), M, N, K, x.stride(0), w.stride(0), splits,
                                            _ptr(status), ctypes.byref(rs), _stream())
        kernels = 2 if splits > 1 else 1
    if st == -2:
        return False
    _check(st, "gemm_qkv_rope", kernels=kernels)
    return True


def sink_flag(sink) -> int:
    return 0 if sink is None or sink is False else 1


def sink_values(sink, n_heads: int) -> Optional[torch.Tensor]:
    """A sink is False / None (none), True (one more key of score 0) or a float32 tensor with every head's score."""
    if not isinstance(sink, torch.Tensor):
        return None
    if sink.dtype != torch.float32 or sink.numel() != n_heads or not sink.is_contiguous():
        raise KernelError("attention: the sink needs one float32 score per head")
    return sink


def attention_simt(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, token_seq: torch.Tensor,
                   token_pos: torch.Tensor, table: torch.Tensor, n_heads: int, scale: float, window: int,
                   status: Optional[torch.Tensor], out: Optional[torch.Tensor] = None, softcap: float = 0.0, sink=False,
                   values_in_keys: int = 0) -> torch.Tensor:
    """``softcap``: scores become cap * tanh(score / cap) after the scale (0 = no cap).  The value pages may
    have a head size of their own; the output is then [T, n_heads * that size].  ``sink``: one more key of score 0
    that carries no value (the weights are exp(s_j) / (1 + sum exp(s_j))); a float32 tensor [n_heads] instead of True gives
    every head's sink a score of its own (not scaled).  ``values_in_keys`` = n > 0: a key row's
    leading n columns are its value (``v_pages`` is not read)."""
    _need(q, "q")
    _need(k_pages, "k_pages")
    _need(table, "table", torch.int32)
    n_pages, nkv, page_size, hd = k_pages.shape
    T = q.shape[0]
    if values_in_keys:
        if not 0 < values_in_keys <= hd:
            raise KernelError("attention: the values cannot be wider than the key rows they lie in")
        v_pages, hdv, ldv = k_pages, int(values_in_keys), hd
    else:
        _need(v_pages, "v_pages")
        hdv = ldv = v_pages.shape[3]
    if q.shape[1] != n_heads * hd or v_pages.shape[:3] != k_pages.shape[:3] or v_pages.dtype != k_pages.dtype:
        raise KernelError("attention: q or the value pages have the wrong shape")
    if out is None:
        out = torch.empty((T, n_heads * hdv), dtype=q.dtype, device=q.device)
    _work(f"attention_simt {T}x{n_heads}", _nbytes(q, out))
    _check(lib().ik_attention_simt(_ptr(q), _code(q), _ptr(k_pages), _ptr(v_pages), _code(k_pages), _ptr(out),
                                   _code(out), _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), T,
                                   n_heads, nkv, hd, hdv, ldv, scale, softcap, window, sink_flag(sink), _ptr(sink_values(sink, n_heads)),
                                   page_size, n_pages, _ptr(status), _stream()),
           "attention_simt")
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out_dtype: torch.dtype,
              rows_in: Optional[torch.Tensor] = None, into: Optional[torch.Tensor] = None, mult: float = 1.0) -> torch.Tensor:
    """y = (x - mean) / sqrt(var + eps) * weight + bias per row, in float.  Returns y in ``out_dtype``, or, when
    ``into`` (float, the shape of x) is given, adds ``mult * y`` to it and returns it."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(bias, "bias", torch.float32)
    d = x.shape[-1]
    if weight.numel() != d or bias.numel() != d:
        raise KernelError(f"layernorm: weight and bias need {d} elements")
    rows = x.numel() // d if rows_in is None else rows_in.numel()
    if rows_in is not None:
        _need(rows_in, "rows_in", torch.int32)
    out = None
    if into is not None:
        _need(into, "into", torch.float32)
        if into.shape != x.shape or rows_in is not None:
            raise KernelError("layernorm: the stream to add to must have the input's shape")
    else:
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
    _work(f"layernorm{' +add' if into is not None else ''} {rows}x{d}", rows * d * (12 if into is not None else 4 + out.element_size()))
    _check(lib().ik_layernorm(_ptr(x), _ptr(rows_in), _ptr(weight), _ptr(bias), _ptr(out), _code(out) if out is not None else F32,
                              _ptr(into), mult, rows, d, eps, _stream()), "layernorm")
    return into if into is not None else out


def add_(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """y += x (float, equal shapes)."""
    _need(y, "y", torch.float32)
    _need(x, "x", torch.float32)
    if y.shape != x.shape:
        raise KernelError("add: shapes differ")
    _work(f"add {y.numel()}", 12 * y.numel())
    _check(lib().ik_add(_ptr(y), _ptr(x), y.numel(), _stream()), "add")
    return y


def conv_rope_append(qkv: torch.Tensor, conv_w: Optional[torch.Tensor], ring: Optional[torch.Tensor], slots: torch.Tensor,
                     cu_seqlens: torch.Tensor, kv_lens: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor,
                     v_pages: torch.Tensor, token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                     inv_freq: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, rotary_dim: int, pairing: int,
                     write_cache: bool, status: Optional[torch.Tensor]) -> None:
    """Short causal convolution over time on the projected q, k, v (``conv_w`` [taps, channels], tap-major; None = no
    convolution), rotary encoding of q and k, append of k and v to the pages.  ``ring`` [max_slots, taps, channels]
    holds each sequence's last projected values and is brought up to date."""
    _need(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages")
    _need(table, "table", torch.int32)
    n_pages, nkv, page_size, hd = k_pages.shape
    hdv = v_pages.shape[3]
    T, ctot = qkv.shape
    taps = 0
    if conv_w is not None:
        _need(conv_w, "conv_w", torch.float32)
        taps = conv_w.shape[0]
        if conv_w.shape[1] != ctot:
            raise KernelError("conv_rope_append: one row of channels per tap is needed")
        if taps > 1:
            _need(ring, "ring", torch.float32)
            if tuple(ring.shape[1:]) != (taps, ctot):
                raise KernelError("conv_rope_append: the ring has the wrong shape")
    if nkv != n_kv_heads or ctot != (n_heads + nkv) * hd + nkv * hdv or v_pages.shape[:3] != k_pages.shape[:3] \
            or v_pages.dtype != k_pages.dtype or q_out.shape != (T, n_heads * hd):
        raise KernelError("conv_rope_append: the sizes do not fit together")
    _work(f"conv_rope_append {T}", _nbytes(qkv, q_out) + T * nkv * (hd + hdv) * k_pages.element_size())
    _check(lib().ik_conv_rope_append(_ptr(qkv), _ptr(conv_w), _ptr(ring) if taps > 1 else 0, _ptr(slots), _ptr(cu_seqlens),
                                     _ptr(kv_lens), _ptr(q_out), _code(q_out), _ptr(k_pages), _ptr(v_pages), _code(k_pages),
                                     _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), _ptr(inv_freq), T,
                                     slots.numel(), n_heads, nkv, hd, hdv, rotary_dim, pairing, taps, page_size, n_pages,
                                     1 if write_cache else 0, _ptr(status), _stream()), "conv_rope_append", kernels=2 if taps > 1 else 1)


MOE_SCORES = {"softmax": 0, "sigmoid": 1}


def moe_route(logits: torch.Tensor, top: int, n_groups: int = 0, keep: int = 0, renorm: bool = False, score: str = "softmax"):
    """Scores over the experts (``score``: the softmax over all logits, or the sigmoid of each by itself) and the ``top`` best among the ``keep`` best of ``n_groups`` groups of
    neighbours (0 groups: among all).  Returns (chosen int32 [T, top], weights float [T, top])."""
    _need(logits, "logits", torch.float32)
    T, E = logits.shape
    chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _work(f"moe_route {T}x{E}", _nbytes(logits, chosen, weight))
    _check(lib().ik_moe_route(_ptr(logits), _ptr(chosen), _ptr(weight), T, E, top, n_groups, keep, 1 if renorm else 0,
                              MOE_SCORES[score], _stream()), "moe_route")
    return chosen, weight


def moe_router(x: torch.Tensor, router: torch.Tensor, top: int, n_groups: int = 0, keep: int = 0, renorm: bool = False,
               score: str = "softmax"):
    """The router's logits ``x router^T`` (float products and sums, whatever type ``x`` has) and the routing of
    ``moe_route``, in one kernel.  Returns (chosen int32 [T, top], weights float [T, top]), or None when the kernel does
    not take these sizes (the caller forms the logits with a product and routes them)."""
    _need(x, "x", contiguous=False)
    _need(router, "router", torch.float32)
    T, K = x.shape
    E = router.shape[0]
    if router.shape[1] != K or x.stride(1) != 1:
        raise KernelError("moe_router: the sizes do not fit together")
    chosen = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((T, top), dtype=torch.float32, device=x.device)
    _work(f"moe_router {T}x{E}x{K}", T * K * x.element_size() + E * K * 4 + 8 * T * top, 2 * T * E * K)
    st = lib().ik_moe_router(_ptr(x), _code(x), _ptr(router), _ptr(chosen), _ptr(weight), T, K, E, top, n_groups, keep,
                             1 if renorm else 0, MOE_SCORES[score], x.stride(0), _stream())
    if st == -2:
        return None
    _check(st, "moe_router")
    return chosen, weight


class MoEPlan:
    """Where a step's (token, choice) pairs sit once grouped by expert: device arrays only."""
    __slots__ = ("offsets", "sorted", "tiles", "n_tiles", "max_tiles", "top", "n_assign", "n_experts")


def moe_sort(chosen: torch.Tensor, n_experts: int) -> MoEPlan:
    _need(chosen, "chosen", torch.int32)
    T, top = chosen.shape
    A = T * top
    bm = lib().ik_moe_tile_rows()
    p = MoEPlan()
    p.top, p.n_assign, p.n_experts = top, A, n_experts
    p.max_tiles = min(A, A // bm + n_experts)
    meta = torch.empty(n_experts + 1 + A + 2 * p.max_tiles + 1, dtype=torch.int32, device=chosen.device)
    p.offsets = meta[:n_experts + 1]
    p.sorted = meta[n_experts + 1:n_experts + 1 + A]
    p.tiles = meta[n_experts + 1 + A:n_experts + 1 + A + 2 * p.max_tiles]
    p.n_tiles = meta[n_experts + 1 + A + 2 * p.max_tiles:]
    _work(f"moe_sort {A}", 8 * A)
    _check(lib().ik_moe_sort(_ptr(chosen), _ptr(p.offsets), _ptr(p.sorted), _ptr(p.tiles), _ptr(p.n_tiles), A, n_experts,
                             p.max_tiles, _stream()), "moe_sort")
    return p


def moe_gemm(mode: int, x: torch.Tensor, w: torch.Tensor, plan: MoEPlan, out_dtype: torch.dtype,
             row_scale: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """Mode 2: ``x`` [T, d] tokens, every row times ``row_scale`` [T, top] of its assignment as it is read, ``w`` [E, ff, d] ->
    ``act`` (one of ``PLAIN_ACTS``) of the product, [A, ff] in sorted order.  Mode 0: ``x`` [T, d] tokens, ``w`` [E, 2 ff, d] (gate j and up j in rows 2j and 2j + 1) -> silu(gate) * up [A, ff] in sorted
    order.  Mode 1: ``x`` [A, ff] in sorted order, ``w`` [E, d, ff] -> [A, d], row t * top + k for token t's choice k."""
    _need(x, "x")
    _need(w, "w")
    E, rows, K = w.shape
    N = rows // 2 if mode == 0 else rows
    if x.shape[1] != K or E != plan.n_experts:
        raise KernelError("moe_gemm: the sizes do not fit together")
    out = torch.empty((plan.n_assign, N), dtype=out_dtype, device=x.device)
    A = plan.n_assign
    _work(f"moe_gemm{mode} {A}x{rows}x{K}", A * K * x.element_size() + min(E, A) * rows * K * w.element_size() + A * N * out.element_size(),
          2 * A * rows * K)
    _check(lib().ik_moe_gemm(mode, _ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), _ptr(plan.offsets),
                             _ptr(plan.sorted), _ptr(plan.tiles), _ptr(plan.n_tiles), plan.max_tiles, plan.top, N, K,
                             x.stride(0), out.stride(0), _ptr(row_scale), PLAIN_ACTS[act] if act is not None else 0, _stream()), "moe_gemm")
    return out


class MoEPaddedPlan:
    """A step's (token, choice) pairs in padded order: every expert's rows start at a multiple of the tile height."""
    __slots__ = ("row_of", "src_token", "src_assign", "tile_group", "n_tiles", "bn", "rows", "top", "n_experts")


def moe_sort_padded(chosen: torch.Tensor, n_experts: int, bn: int) -> MoEPaddedPlan:
    _need(chosen, "chosen", torch.int32)
    T, top = chosen.shape
    A = T * top
    p = MoEPaddedPlan()
    p.top, p.n_experts, p.bn = top, n_experts, bn
    p.n_tiles = min(A, A // bn + n_experts)              # a tile holds at least one row; an expert wastes less than one tile
    p.rows = p.n_tiles * bn
    meta = torch.empty(A + 2 * p.rows + p.n_tiles, dtype=torch.int32, device=chosen.device)
    p.row_of, p.src_token, p.tile_group = meta[:A], meta[A:A + p.rows], meta[A + p.rows:A + p.rows + p.n_tiles]
    p.src_assign = meta[A + p.rows + p.n_tiles:]
    _work(f"moe_sort_padded {A}", 8 * A + 4 * p.rows)
    _check(lib().ik_moe_sort_padded(_ptr(chosen), _ptr(p.row_of), _ptr(p.src_token), _ptr(p.tile_group), A, n_experts, top, bn,
                                    p.n_tiles, _ptr(p.src_assign), _stream()), "moe_sort_padded")
    return p


def moe_gather(x: torch.Tensor, plan: MoEPaddedPlan, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The tokens' activations in padded order [rows, d] (bfloat16; padding rows zero).  ``weight`` [T, top] float: every row
    is multiplied by the weight of its assignment (in float, rounded once)."""
    _need(x, "x", torch.bfloat16)
    d = x.shape[1]
    out = torch.empty((plan.rows, d), dtype=torch.bfloat16, device=x.device)
    _work(f"moe_gather {plan.rows}x{d}", 4 * plan.rows * d)
    if weight is not None:
        _need(weight, "weight", torch.float32)
        _check(lib().ik_moe_gather_scaled(_ptr(x), _ptr(plan.src_token), _ptr(plan.src_assign), _ptr(weight), _ptr(out), plan.rows, d,
                                          _stream()), "moe_gather")
        return out
    _check(lib().ik_moe_gather(_ptr(x), _ptr(plan.src_token), _ptr(out), plan.rows, d, _stream()), "moe_gather")
    return out


def gemm_tcgen05_grouped(x: torch.Tensor, w: torch.Tensor, plan: MoEPaddedPlan, out_dtype: torch.dtype, swiglu: bool = False,
                         status: Optional[torch.Tensor] = None, act: Optional[str] = None) -> Optional[torch.Tensor]:
    """``x`` [rows, K] in padded order, ``w`` [E * N, K]: the stacked matrices of the experts; token tile i of ``plan.bn``
    rows multiplies matrix ``plan.tile_group[i]``.  Returns [rows, N] (N / 2 with the SwiGLU epilogue; rows of unused
    tiles are left as they are), or None when the tcgen05 kernel does not take these sizes."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0] // plan.n_experts
    if w.shape[1] != K or M != plan.rows or w.shape[0] != N * plan.n_experts:
        raise KernelError("gemm_tcgen05_grouped: the sizes do not fit together")
    if K % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or (swiglu and N % 2):
        return None
    n_out = N // 2 if swiglu else N
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    used = min(M, plan.rows)
    _work(f"gemm_tcgen05 grouped{' +swiglu' if swiglu else ''} {used}x{N}x{K}", 2 * (used * K + min(plan.n_experts, plan.n_tiles) * N * K) + used * n_out * out.element_size(),
          2 * used * N * K)
    st = lib().ik_gemm_tcgen05_grouped(_ptr(x), _ptr(w), _ptr(out), _code(out), _ptr(plan.tile_group), plan.n_experts, plan.bn,
                                       M, N, K, x.stride(0), w.stride(0), out.stride(0), 1 if swiglu else _act_code(act),
                                       _ptr(status), _stream())
    if st == -2:
        return None
    _check(st, "gemm_tcgen05_grouped")
    return out


def moe_combine(parts: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_of: Optional[torch.Tensor] = None, unweighted: bool = False) -> torch.Tensor:
    """y[t] = sum_k weight[t, k] * parts[row_of[t * top + k]] (``row_of`` None: row t * top + k).  ``unweighted``: a plain sum
    (``weight`` then only gives the shape)."""
    _need(parts, "parts", torch.float32)
    _need(weight, "weight", torch.float32)
    T, top = weight.shape
    d = parts.shape[1]
    if row_of is None and parts.shape[0] != T * top:
        raise KernelError("moe_combine: one row per (token, choice) is needed")
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=parts.device)
    _work(f"moe_combine {T}x{d}", _nbytes(parts, out))
    _check(lib().ik_moe_combine(_ptr(parts), 0 if unweighted else _ptr(weight), _ptr(row_of), _ptr(out), T, top, d, _stream()),
           "moe_combine")
    return out


def wait_records() -> str:
    """Where the first wait of each tensor-core module gave up since the last call (read and cleared): text for an
    error message, empty if none did."""
    found = []
    rec = (ctypes.c_int * 4)()
    takers = [("matrix product", lib().ik_gemm_tcgen05_take_wait_record)]
    from . import attention_bf16
    for hd, m in attention_bf16._modules.items():
        takers.append((f"attention (head size {hd})", m.ik_attn_take_wait_record))
    for name, take in takers:
        if take(rec) == 0 and rec[0] != 0:
            found.append(f"{name}: wait site {rec[0]}, block {rec[1]}, count {rec[2]}, parity {rec[3]}")
    return "; ".join(found)


def selftest_wait_expires(status: torch.Tensor, limit_ns: int = 1_000_000) -> torch.Tensor:
    """Runs the kernel library's check of its bounded waits: waits that nothing satisfies, with a limit of
    ``limit_ns`` (at most 10 ms).  Returns int32 [6]: see gemm_tcgen05.cu."""
    result = torch.full((6,), -1, dtype=torch.int32, device=status.device)
    never = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(lib().ik_selftest_wait_expires(_ptr(status), _ptr(result), _ptr(never), limit_ns, _stream()), "selftest_wait_expires")
    return result


def tcgen05_issue_rate(n: int, per_commit: int, issuers: int, status: torch.Tensor) -> float:
    """Cycles of the SM clock per tcgen05 product instruction (128 rows, 16 k, ``n`` tokens) when ``issuers`` threads (1 or
    2) issue them back to back, ``per_commit`` between commits, and nothing else runs: what the issuing thread costs.
    With two threads the figure is per thread; together they issue twice as many."""
    out = torch.zeros(2, dtype=torch.int64, device=status.device)
    _check(lib().ik_gemm_tcgen05_issue_rate(n, per_commit, issuers, _ptr(out), _ptr(status), _stream()), "tcgen05_issue_rate")
    cycles, fine = (int(v) for v in out.tolist())
    if not fine:
        raise KernelError("tcgen05_issue_rate: a wait ran out")
    return cycles / (64 * per_commit)


_argmax_scratch = {}


def argmax_scratch(device, fresh: bool = False) -> torch.Tensor:
    """Scratch of the split argmax (counters and per-slice bests), zeroed once; the kernel leaves it as it found
    it.  Launches that share one must follow one another in one stream: by default there is one per (device,
    stream); ``fresh`` makes one for a caller that keeps its own (a captured graph)."""
    if fresh:
        return torch.zeros(lib().ik_argmax_scratch_bytes() // 4, dtype=torch.int32, device=device)
    key = (str(torch.device(device)), _stream())
    t = _argmax_scratch.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("argmax: no scratch exists for this stream yet and none can be made during a capture; "
                              "pass one made with argmax_scratch(device, fresh=True)")
        t = _argmax_scratch[key] = torch.zeros(lib().ik_argmax_scratch_bytes() // 4, dtype=torch.int32, device=device)
    return t


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of each row's largest value (the lowest index among equals)."""
    _need(logits, "logits", torch.float32, contiguous=False)
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if scratch is None:
        scratch = argmax_scratch(logits.device)
    _work(f"argmax {rows}x{V}", rows * V * 4)
    _check(lib().ik_argmax(_ptr(logits), logits.stride(0), _ptr(out), rows, V, _ptr(scratch), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repetition_penalty: float,
           recent: Optional[torch.Tensor], seed: int, streams: torch.Tensor, counters: torch.Tensor,
           out: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(streams, "streams", torch.int32)
    _need(counters, "counters", torch.int32)
    rows, V = logits.shape
    n_recent = 0
    if recent is not None:
        _need(recent, "recent", torch.int32)
        n_recent = recent.shape[1]
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if work is None:
        work = torch.empty((rows, V), dtype=torch.float32, device=logits.device)
    _work(f"sample {rows}x{V}", 3 * rows * V * 4)
    _check(lib().ik_sample(_ptr(logits), logits.stride(0), _ptr(work), _ptr(out), rows, V, temperature, top_k, top_p,
                           repetition_penalty, _ptr(recent), n_recent, seed & 0xFFFFFFFFFFFFFFFF, _ptr(streams),
                           _ptr(counters), _stream()), "sample")
    return out


# ---------------------------------------------------------------------------------------------
# Norm behind a sublayer, casts, the gated activation with parameters, logit scale and cap
def rmsnorm_add(y: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor, scale: Optional[torch.Tensor] = None,
                mult: float = 1.0, copy: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += mult * scale * rmsnorm(y) * weight (``scale``: a vector or None).  ``copy`` (the residual's shape, any
    kernel type) receives the new residual."""
    _need(y, "y", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(residual, "residual", torch.float32)
    d = y.shape[-1]
    if weight.numel() != d or residual.shape != y.shape or (scale is not None and scale.numel() != d):
        raise KernelError("rmsnorm_add: the sizes do not fit together")
    if scale is not None:
        _need(scale, "scale", torch.float32)
    if copy is not None:
        _need(copy, "copy")
        if copy.shape != y.shape:
            raise KernelError("rmsnorm_add: the copy must have the residual's shape")
    rows = y.numel() // d
    _work(f"rmsnorm +add {rows}x{d}", rows * d * 12 + _nbytes(copy))
    _check(lib().ik_rmsnorm_add(_ptr(y), _ptr(weight), _ptr(scale), _ptr(residual), _ptr(copy), _code(copy) if copy is not None else F32,
                                rows, d, eps, mult, _stream()), "rmsnorm_add")
    return residual


def cast(x: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A float matrix (rows may be wider apart than their length: a column range) in another type, rows contiguous."""
    _need(x, "x", torch.float32, contiguous=False)
    rows, cols = x.shape
    if x.stride(1) != 1:
        raise KernelError("cast: rows must be contiguous")
    if out is None:
        out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
    _need(out, "out")
    _work(f"cast {rows}x{cols}", rows * cols * (4 + out.element_size()))
    _check(lib().ik_cast(_ptr(x), x.stride(0), _ptr(out), _code(out), cols, rows, cols, _stream()), "cast")
    return out


def scale_softcap_(v: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """v <- v * scale, then cap * tanh(v / cap) when cap > 0 (float, in place)."""
    _need(v, "v", torch.float32)
    _work(f"scale_softcap {v.numel()}", 8 * v.numel())
    _check(lib().ik_scale_softcap(_ptr(v), v.numel(), scale, cap, _stream()), "scale_softcap")
    return v


def glu_act(gate_up: torch.Tensor, out_dtype: torch.dtype, alpha: float, limit: float, shift: float,
            out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """g <- min(g, limit), u <- clamp(u, -limit, limit) (limit > 0); g * sigmoid(alpha g) * (u + shift)."""
    _need(gate_up, "gate_up", torch.float32)
    T, ff2 = gate_up.shape
    if ff2 % 2:
        raise KernelError("glu_act: the input needs an even number of columns (gate then up)")
    if out is None:
        out = torch.empty((T, ff2 // 2), dtype=out_dtype, device=gate_up.device)
    _work(f"glu_act {T}x{ff2 // 2}", _nbytes(gate_up, out))
    _check(lib().ik_glu_act(_ptr(gate_up), _ptr(out), _code(out), T, ff2 // 2, 1 if interleaved else 0, alpha, limit, shift, _stream()),
           "glu_act")
    return out


# ---------------------------------------------------------------------------------------------
# Mixers with a state of fixed size
def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], ring: Optional[torch.Tensor], ctx,
                out_dtype: torch.dtype, act: bool = True) -> torch.Tensor:
    """Causal convolution over time per channel with bias and silu.  ``x`` [T, C] float (rows may be a column range),
    ``w`` [taps, C] tap-major, ``ring`` [max_slots, taps, C] float: each sequence's last inputs, brought up to date."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(w, "w", torch.float32)
    T, C = x.shape
    taps = w.shape[0]
    if w.shape[1] != C or x.stride(1) != 1 or (bias is not None and bias.numel() != C):
        raise KernelError("causal_conv: the sizes do not fit together")
    if taps > 1:
        _need(ring, "ring", torch.float32)
        if tuple(ring.shape[1:]) != (taps, C):
            raise KernelError("causal_conv: the ring has the wrong shape")
    out = torch.empty((T, C), dtype=out_dtype, device=x.device)
    _work(f"causal_conv {T}x{C}", T * C * (4 + out.element_size()))
    _check(lib().ik_causal_conv(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(ring) if taps > 1 else 0, _ptr(ctx.slots),
                                _ptr(ctx.cu_seqlens), _ptr(ctx.kv_lens), _ptr(ctx.token_seq), _ptr(ctx.token_pos), _ptr(out),
                                _code(out), T, ctx.n_seqs, C, taps, 1 if act else 0, 1 if ctx.is_decode else 0, _stream()),
           "causal_conv", kernels=1 if ctx.is_decode or taps == 1 else 2)
    return out


def selective_scan(u: torch.Tensor, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], A: torch.Tensor, bc: torch.Tensor,
                   b_off: int, c_off: int, D: Optional[torch.Tensor], z: Optional[torch.Tensor], state: torch.Tensor, ctx,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """The selective scan over the step's tokens, sequence by sequence.  ``u`` [T, inner], ``dt_raw`` [T, inner] float
    (before bias and softplus), ``A`` [inner, N] float (negative), B and C = columns ``b_off``.. and ``c_off``.. of ``bc``,
    ``z`` [T, inner] float (rows may be a column range) for the gate y * silu(z), ``state`` [max_slots, 2, inner, N] float."""
    _need(u, "u")
    _need(dt_raw, "dt_raw", torch.float32)
    _need(A, "A", torch.float32)
    _need(bc, "bc", torch.float32, contiguous=False)
    _need(state, "state", torch.float32)
    T, inner = u.shape
    N = A.shape[1]
    if A.shape[0] != inner or dt_raw.shape != (T, inner) or tuple(state.shape[1:]) != (2, inner, N) or bc.stride(1) != 1 \
            or max(b_off, c_off) + N > bc.shape[1]:
        raise KernelError("selective_scan: the sizes do not fit together")
    ldz = 0
    if z is not None:
        _need(z, "z", torch.float32, contiguous=False)
        if z.shape != (T, inner) or z.stride(1) != 1:
            raise KernelError("selective_scan: the gate has the wrong shape")
        ldz = z.stride(0)
    out = torch.empty((T, inner), dtype=out_dtype, device=u.device)
    _work(f"selective_scan {T}x{inner}x{N}", T * inner * (u.element_size() + 8 + out.element_size()) + 8 * ctx.n_seqs * inner * N,
          9 * T * inner * N)
    st = lib().ik_selective_scan(_ptr(u), _code(u), _ptr(dt_raw), _ptr(dt_bias), _ptr(A), _ptr(bc), bc.stride(0), b_off, c_off,
                                 _ptr(D), _ptr(z), ldz, _ptr(state), _ptr(ctx.slots), _ptr(ctx.cu_seqlens), _ptr(ctx.kv_lens),
                                 _ptr(out), _code(out), T, ctx.n_seqs, inner, N, 1 if ctx.is_decode else 0, _stream())
    _check(st, "selective_scan")
    return out


def decay_attention(p: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor, state: torch.Tensor, ctx,
                    n_heads: int, dk: int, dv: int, act: int = 1) -> torch.Tensor:
    """Linear attention with one constant decay per head: S <- a S + k v^T, o = S^T q, over the step's tokens.  q, k, v
    are column ranges of ``p`` (float), passed through silu when ``act`` (2: silu with the hardware's approximate
    exponential and reciprocal, for the 16-bit path).  ``state`` [max_slots, 2, heads, dv, dk] float (column by column).
    Returns float [T, heads * dv]."""
    _need(p, "p", torch.float32, contiguous=False)
    _need(decay, "decay", torch.float32)
    _need(state, "state", torch.float32)
    T = p.shape[0]
    if decay.numel() != n_heads or tuple(state.shape[1:]) != (2, n_heads, dk, dv) or p.stride(1) != 1 \
            or max(q_off + n_heads * dk, k_off + n_heads * dk, v_off + n_heads * dv) > p.shape[1]:
        raise KernelError("decay_attention: the sizes do not fit together")
    out = torch.empty((T, n_heads * dv), dtype=torch.float32, device=p.device)
    _work(f"decay_attention {T}x{n_heads}x{dk}x{dv}", T * n_heads * (2 * dk + 2 * dv) * 4 + 8 * ctx.n_seqs * n_heads * dk * dv,
          4 * T * n_heads * dk * dv)
    _check(lib().ik_decay_attention(_ptr(p), p.stride(0), q_off, k_off, v_off, _ptr(decay), _ptr(state), _ptr(ctx.slots),
                                    _ptr(ctx.cu_seqlens), _ptr(ctx.kv_lens), _ptr(out), T, ctx.n_seqs, n_heads, dk, dv,
                                    int(act), 1 if ctx.is_decode else 0, _stream()), "decay_attention")
    return out


# ---------------------------------------------------------------------------------------------
# Around an attention core whose projections come out of one wide product
def norm_rope_append(p: torch.Tensor, q_off: int, k_off: int, v_off: int, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                     eps: float, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, token_seq: torch.Tensor,
                     token_pos: torch.Tensor, table: torch.Tensor, inv_freq: Optional[torch.Tensor], magnitude: float,
                     n_heads: int, rotary_dim: int, pairing: int, write_cache: bool, status: Optional[torch.Tensor],
                     per_head: bool = False, bias: Optional[torch.Tensor] = None, v_norm: bool = False) -> None:
    """``bias``: a float vector over ``p``'s columns, added to q, k and v as they are read.  ``v_norm``: every value head is
    divided by the root mean square of its own values (``eps`` inside the root) before it is stored.
    RMS norm of q and of k over their whole projections (``q_w``, ``k_w``: weights of that size; None = no norm;
    ``per_head``: every head over its own values, with a weight of one head's size that the heads share),
    rotation of each head's leading ``rotary_dim`` dimensions with cos and sin times ``magnitude``, q to ``q_out``,
    k and v into the pages.  q, k, v are column ranges of ``p`` (float)."""
    _need(p, "p", torch.float32, contiguous=False)
    _need(q_out, "q_out")
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages")
    _need(table, "table", torch.int32)
    n_pages, nkv, page_size, hd = k_pages.shape
    hdv = v_pages.shape[3]
    T = p.shape[0]
    if p.stride(1) != 1 or q_out.shape != (T, n_heads * hd) or v_pages.shape[:3] != k_pages.shape[:3] or v_pages.dtype != k_pages.dtype \
            or max(q_off + n_heads * hd, k_off + nkv * hd, v_off + nkv * hdv) > p.shape[1] \
            or (q_w is not None and q_w.numel() != (hd if per_head else n_heads * hd)) \
            or (k_w is not None and k_w.numel() != (hd if per_head else nkv * hd)) \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() < max(q_off + n_heads * hd, k_off + nkv * hd, v_off + nkv * hdv))):
        raise KernelError("norm_rope_append: the sizes do not fit together")
    _work(f"norm_rope_append {T}", T * ((n_heads + nkv) * hd + nkv * hdv) * 4 + _nbytes(q_out) + T * nkv * (hd + hdv) * k_pages.element_size())
    _check(lib().ik_norm_rope_append(_ptr(p), p.stride(0), q_off, k_off, v_off, _ptr(q_w), _ptr(k_w), eps, _ptr(q_out), _code(q_out),
                                     _ptr(k_pages), _ptr(v_pages), _code(k_pages), _ptr(token_seq), _ptr(token_pos), _ptr(table),
                                     table.stride(0), _ptr(inv_freq), magnitude, T, n_heads, nkv, hd, hdv, rotary_dim, pairing,
                                     page_size, n_pages, 1 if write_cache else 0, 1 if per_head else 0, _ptr(bias), 1 if v_norm else 0, _ptr(status),
                                     _stream()), "norm_rope_append")


def head_gate(att: torch.Tensor, p: Optional[torch.Tensor], g_off: int, out: torch.Tensor, n_heads: int, mult: float = 1.0,
              wide: bool = False) -> torch.Tensor:
    """out[t, h, :] = att[t, h, :] * sigmoid(p[t, g_off + h]) * mult (``p`` None: no gate); ``out`` may be a column range of
    a wider matrix.  ``wide``: the gate has one number per value, p[t, g_off + column]."""
    _need(att, "att")
    _need(out, "out", att.dtype, contiguous=False)
    T, cols = att.shape
    ldp = 0
    if p is not None:
        _need(p, "p", torch.float32, contiguous=False)
        if p.stride(1) != 1 or g_off + (cols if wide else n_heads) > p.shape[1]:
            raise KernelError("head_gate: the gate has the wrong shape")
        ldp = p.stride(0)
    if cols % n_heads or out.shape != att.shape or out.stride(1) != 1:
        raise KernelError("head_gate: the sizes do not fit together")
    _work(f"head_gate {T}x{cols}", 2 * _nbytes(att))
    _check(lib().ik_head_gate(_ptr(att), _ptr(p), ldp, g_off, _ptr(out), _code(att), out.stride(0), T, n_heads,
                              cols // n_heads, mult, 1 if wide else 0, _stream()), "head_gate")
    return out


def gated_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, p: Optional[torch.Tensor], g_off: int, out: torch.Tensor,
                  mult: float = 1.0) -> torch.Tensor:
    """out = rmsnorm(x) * weight * sigmoid(p[:, g_off : g_off + d]) * mult (no gate when ``p`` is None); ``out`` may be a column
    range of a wider matrix."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out", contiguous=False)
    rows, d = x.shape
    ldp = 0
    if p is not None:
        _need(p, "p", torch.float32, contiguous=False)
        if p.stride(1) != 1 or g_off + d > p.shape[1]:
            raise KernelError("gated_rmsnorm: the gate has the wrong shape")
        ldp = p.stride(0)
    if weight.numel() != d or out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("gated_rmsnorm: the sizes do not fit together")
    _work(f"gated_rmsnorm {rows}x{d}", rows * d * (8 + out.element_size()))
    _check(lib().ik_gated_rmsnorm(_ptr(x), _ptr(weight), _ptr(p), ldp, g_off, _ptr(out), _code(out), out.stride(0), rows, d, eps,
                                  mult, _stream()), "gated_rmsnorm")
    return out


# ---------------------------------------------------------------------------------------------
# A layer-scaled sublayer result into the stream (with the next norm), the ungated feed-forward's activation
def scale_add_norm(y: torch.Tensor, scale: Optional[torch.Tensor], residual: torch.Tensor, weight: Optional[torch.Tensor] = None,
                   eps: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """residual += scale * y (``scale``: a vector or None).  With ``weight``: returns rmsnorm(new residual) * weight in
    ``out_dtype``, formed in the same pass over the rows."""
    _need(y, "y", torch.float32)
    _need(residual, "residual", torch.float32)
    d = y.shape[-1]
    if residual.shape != y.shape or (scale is not None and scale.numel() != d) or (weight is not None and weight.numel() != d):
        raise KernelError("scale_add_norm: the sizes do not fit together")
    if scale is not None:
        _need(scale, "scale", torch.float32)
    rows = y.numel() // d
    out = None
    if weight is not None:
        _need(weight, "weight", torch.float32)
        out = torch.empty((rows, d), dtype=out_dtype or torch.float32, device=y.device)
    _work(f"scale_add{' +rmsnorm' if weight is not None else ''} {rows}x{d}", rows * d * 12 + _nbytes(out))
    _check(lib().ik_scale_add_norm(_ptr(y), _ptr(scale), _ptr(residual), _ptr(weight), _ptr(out), _code(out) if out is not None else F32,
                                   rows, d, eps, _stream()), "scale_add_norm")
    return out


PLAIN_ACTS = {"relu2": 0, "gelu_tanh": 1, "tanh": 2}


def plain_act(x: torch.Tensor, out_dtype: torch.dtype, act: str) -> torch.Tensor:
    """relu(x)^2 (``relu2``) or the tanh form of gelu (``gelu_tanh``), float in, ``out_dtype`` out."""
    _need(x, "x", torch.float32)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _work(f"plain_act {x.numel()}", _nbytes(x, out))
    _check(lib().ik_plain_act(_ptr(x), _ptr(out), _code(out), x.numel(), PLAIN_ACTS[act], _stream()), "plain_act")
    return out


def gemm_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One product per head in one launch: out[:, h, :] = x[:, h, :] @ w[h]^T.  ``x`` [T, H, K] and ``out`` [T, H, N] may be
    column ranges of wider rows (their last dimension contiguous), ``w`` [H, N, K]; float accumulation in ascending k."""
    _need(x, "x", contiguous=False)
    _need(w, "w")
    _need(out, "out", contiguous=False)
    T, H, K = x.shape
    if w.shape[0] != H or w.shape[2] != K or out.shape != (T, H, w.shape[1]) or x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("gemm_heads: the sizes do not fit together")
    N = w.shape[1]
    _work(f"gemm_heads {H}x{T}x{N}x{K}", _nbytes(w) + T * H * (K * x.element_size() + N * out.element_size()), 2 * T * H * N * K)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        # the heads as a batch of the warp-level tensor-core product
        st = lib().ik_gemm_bf16_mma_batched(_ptr(x), _ptr(w), _ptr(out), _code(out), T, N, K, x.stride(0), K, out.stride(0), H,
                                            x.stride(1), N * K, out.stride(1), _stream())
        if st != -2:
            _check(st, "gemm_heads")
            return out
    _check(lib().ik_gemm_simt_batched(_ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), T, N, K, x.stride(0), K, out.stride(0),
                                      H, x.stride(1), N * K, out.stride(1), _stream()), "gemm_heads")
    return out


# ---------------------------------------------------------------------------------------------
# The gated delta rule
def delta_prepare(u: torch.Tensor, q_off: int, k_off: int, p: torch.Tensor, b_off: int, a_off: int, A_log: Optional[torch.Tensor],
                  dt_bias: Optional[torch.Tensor], n_qk_heads: int, dk: int, n_heads: int, q_mult: float, unit_eps: float) -> torch.Tensor:
    """In place: every q and k head of ``u`` (float, behind convolution and activation) becomes a unit vector, q times
    ``q_mult``.  Returns float [T, 2, heads]: the steps sigmoid(p_b) and the decays exp(-exp(A_log) softplus(p_a + dt_bias)).
    ``a_off`` < 0: no decay per head is formed (the second row is not written)."""
    _need(u, "u", torch.float32)
    _need(p, "p", torch.float32, contiguous=False)
    if a_off >= 0:
        _need(A_log, "A_log", torch.float32)
        _need(dt_bias, "dt_bias", torch.float32)
    T = u.shape[0]
    if p.stride(1) != 1 or max(b_off, a_off) + n_heads > p.shape[1] or max(q_off, k_off) + n_qk_heads * dk > u.shape[1] \
            or (a_off >= 0 and (A_log.numel() != n_heads or dt_bias.numel() != n_heads)):
        raise KernelError("delta_prepare: the sizes do not fit together")
    bg = torch.empty((T, 2, n_heads), dtype=torch.float32, device=u.device)
    _work(f"delta_prepare {T}", 2 * T * 2 * n_qk_heads * dk * 4)
    _check(lib().ik_delta_prepare(_ptr(u), u.stride(0), q_off, k_off, _ptr(p), p.stride(0), b_off, a_off, _ptr(A_log), _ptr(dt_bias),
                                  _ptr(bg), T, n_qk_heads, dk, n_heads, q_mult, unit_eps, _stream()), "delta_prepare")
    return bg


def delta_rule(u: torch.Tensor, q_off: int, k_off: int, v_off: int, bg: torch.Tensor, state: torch.Tensor, ctx, n_heads: int,
               n_qk_heads: int, dk: int, dv: int) -> torch.Tensor:
    """The gated delta rule over the step's tokens: per head S <- g S; u = b (v - S^T k); S <- S + k u^T; o = S^T q.  q, k
    (``n_qk_heads`` heads, unit vectors) and v are column ranges of ``u`` (float), ``bg`` [T, 2, heads] the steps and decays,
    ``state`` [max_slots, 2, heads, dv, dk] float (column by column).  Returns float [T, heads * dv]."""
    _need(u, "u", torch.float32)
    _need(bg, "bg", torch.float32)
    _need(state, "state", torch.float32)
    T = u.shape[0]
    if tuple(state.shape[1:]) != (2, n_heads, dv, dk) or bg.shape != (T, 2, n_heads) or n_heads % n_qk_heads \
            or max(q_off + n_qk_heads * dk, k_off + n_qk_heads * dk, v_off + n_heads * dv) > u.shape[1]:
        raise KernelError("delta_rule: the sizes do not fit together")
    out = torch.empty((T, n_heads * dv), dtype=torch.float32, device=u.device)
    _work(f"delta_rule {T}x{n_heads}x{dk}x{dv}", T * (2 * n_qk_heads * dk + 2 * n_heads * dv) * 4 + 8 * ctx.n_seqs * n_heads * dk * dv,
          6 * T * n_heads * dk * dv)
    _check(lib().ik_delta_rule(_ptr(u), u.stride(0), q_off, k_off, v_off, _ptr(bg), _ptr(state), _ptr(ctx.slots), _ptr(ctx.cu_seqlens),
                               _ptr(ctx.kv_lens), _ptr(out), T, ctx.n_seqs, n_heads, n_qk_heads, dk, dv, 1 if ctx.is_decode else 0,
                               _stream()), "delta_rule")
    return out


HEAD_GATES = {None: 0, "silu": 1, "sigmoid": 2}


def head_norm_gate_into(x: torch.Tensor, weight: torch.Tensor, eps: float, p: Optional[torch.Tensor], g_off: int, n_heads: int,
                        out: torch.Tensor, gate: Optional[str] = "silu") -> torch.Tensor:
    """``head_norm_gate`` into a matrix the caller owns (contiguous, [T, heads * dv])."""
    return head_norm_gate(x, weight, eps, p, g_off, n_heads, out.dtype, gate, out=out)


def head_norm_gate(x: torch.Tensor, weight: torch.Tensor, eps: float, p: Optional[torch.Tensor], g_off: int, n_heads: int,
                   out_dtype: torch.dtype, gate: Optional[str] = "silu", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of every head of ``x`` [T, heads * dv] over its dv values with one weight of size dv (or one of size
    heads * dv: every head its own), times silu or sigmoid of columns ``g_off``.. of ``p`` (``gate`` None: no gate)."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    T, cols = x.shape
    dv = cols // n_heads
    ldp = 0
    if gate is not None:
        _need(p, "p", torch.float32, contiguous=False)
        if p.stride(1) != 1 or g_off + cols > p.shape[1]:
            raise KernelError("head_norm_gate: the gate has the wrong shape")
        ldp = p.stride(0)
    if cols % n_heads or weight.numel() not in (dv, cols):
        raise KernelError("head_norm_gate: the sizes do not fit together")
    if out is None:
        out = torch.empty((T, cols), dtype=out_dtype, device=x.device)
    _need(out, "out")
    if out.shape != (T, cols):
        raise KernelError("head_norm_gate: the output has the wrong shape")
    _work(f"head_norm_gate {T}x{cols}", T * cols * (8 + out.element_size()))
    _check(lib().ik_head_norm_gate(_ptr(x), _ptr(weight), _ptr(p) if gate is not None else 0, ldp, g_off, _ptr(out), _code(out), T,
                                   n_heads, dv, eps, HEAD_GATES[gate], dv if (weight.numel() == cols and n_heads > 1) else 0, _stream()),
           "head_norm_gate")
    return out


# ---------------------------------------------------------------------------------------------
# Latent attention
def latent_prepare(p: torch.Tensor, q_off: int, c_off: int, c_w: Optional[torch.Tensor], eps: float, q_plain: torch.Tensor,
                   q_full: torch.Tensor, k_pages: torch.Tensor, token_seq: torch.Tensor, token_pos: torch.Tensor, table: torch.Tensor,
                   inv_freq: Optional[torch.Tensor], n_heads: int, dk: int, dr: int, rank: int, write_cache: bool,
                   status: Optional[torch.Tensor]) -> None:
    """From the projections ``p`` (float): every query head's plain part to ``q_plain`` [T, heads, dk], its turning part,
    turned, to the last ``dr`` columns of ``q_full`` [T, heads, rank + dr]; when the layer writes rows, the normed latent
    and the turned shared key part into the token's row of ``k_pages`` [pages, 1, page_size, rank + dr]."""
    _need(p, "p", torch.float32, contiguous=False)
    _need(q_plain, "q_plain")
    _need(q_full, "q_full", q_plain.dtype)
    _need(k_pages, "k_pages")
    _need(table, "table", torch.int32)
    if dr:
        _need(inv_freq, "inv_freq", torch.float32)
    n_pages, nkv, page_size, hd = k_pages.shape
    T = p.shape[0]
    if p.stride(1) != 1 or nkv != 1 or hd != rank + dr or q_plain.shape != (T, n_heads * dk) or q_full.shape != (T, n_heads * hd) \
            or (dr and inv_freq.numel() != dr // 2) or q_off + n_heads * (dk + dr) > p.shape[1] \
            or (write_cache and (c_w is None or c_w.numel() != rank or c_off + hd > p.shape[1])):
        raise KernelError("latent_prepare: the sizes do not fit together")
    _work(f"latent_prepare {T}", T * (n_heads * (dk + dr) * (4 + q_plain.element_size()) + hd * (4 + k_pages.element_size())))
    _check(lib().ik_latent_prepare(_ptr(p), p.stride(0), q_off, c_off, _ptr(c_w), eps, _ptr(q_plain), _ptr(q_full), _code(q_plain),
                                   _ptr(k_pages), _code(k_pages), _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0),
                                   _ptr(inv_freq), T, n_heads, dk, dr, rank, page_size, n_pages, 1 if write_cache else 0,
                                   _ptr(status), _stream()), "latent_prepare")


def latent_append(p: torch.Tensor, c_off: int, c_w: torch.Tensor, eps: float, k_pages: torch.Tensor, token_seq: torch.Tensor,
                  token_pos: torch.Tensor, table: torch.Tensor, rank: int, status: Optional[torch.Tensor]) -> None:
    """The latent alone, for a layer whose queries are made elsewhere and whose rows have no turning part: columns ``c_off``..
    of ``p`` (float), RMS-normed with ``c_w``, into the token's row of ``k_pages`` [pages, 1, page_size, rank]."""
    _need(p, "p", torch.float32, contiguous=False)
    _need(k_pages, "k_pages")
    _need(table, "table", torch.int32)
    _need(c_w, "c_w", torch.float32)
    n_pages, nkv, page_size, hd = k_pages.shape
    T = p.shape[0]
    if p.stride(1) != 1 or nkv != 1 or hd != rank or c_w.numel() != rank or c_off + rank > p.shape[1]:
        raise KernelError("latent_append: the sizes do not fit together")
    _work(f"latent_append {T}", T * rank * (4 + k_pages.element_size()))
    _check(lib().ik_latent_prepare(_ptr(p), p.stride(0), 0, c_off, _ptr(c_w), eps, 0, 0, _code(k_pages), _ptr(k_pages), _code(k_pages),
                                   _ptr(token_seq), _ptr(token_pos), _ptr(table), table.stride(0), 0, T, 0, 0, 0, rank, page_size,
                                   n_pages, 1, _ptr(status), _stream()), "latent_append")


# ---------------------------------------------------------------------------------------------
# Several residual streams per token; norms that join branches
def hyper_start(x: torch.Tensor, n: int) -> torch.Tensor:
    """[T, n, d]: every one of the ``n`` streams a copy of ``x`` [T, d]."""
    _need(x, "x", torch.float32)
    T, d = x.shape
    out = torch.empty((T, n, d), dtype=torch.float32, device=x.device)
    _work(f"hyper_start {T}x{n}x{d}", _nbytes(x, out))
    _check(lib().ik_hyper_start(_ptr(x), _ptr(out), T, n, d, _stream()), "hyper_start")
    return out


def hyper_read(xs: torch.Tensor, a: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows_in: Optional[torch.Tensor] = None) -> torch.Tensor:
    """rmsnorm(sum_s a[s] xs[:, s, :]) * weight for the rows ``rows_in`` names (all without it); ``a`` None: the plain sum."""
    _need(xs, "xs", torch.float32)
    _need(weight, "weight", torch.float32)
    T, n, d = xs.shape
    if weight.numel() != d or (a is not None and (a.numel() != n or a.dtype != torch.float32)):
        raise KernelError("hyper_read: the sizes do not fit together")
    rows = T if rows_in is None else rows_in.numel()
    if rows_in is not None:
        _need(rows_in, "rows_in", torch.int32)
    out = torch.empty((rows, d), dtype=out_dtype, device=xs.device)
    _work(f"hyper_read {rows}x{n}x{d}", rows * d * (4 * n + out.element_size()))
    _check(lib().ik_hyper_read(_ptr(xs), _ptr(rows_in), _ptr(a), _ptr(weight), _ptr(out), _code(out), rows, n, d, eps, _stream()),
           "hyper_read")
    return out


def hyper_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, b: torch.Tensor, a_next: Optional[torch.Tensor] = None,
                w_next: Optional[torch.Tensor] = None, eps: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """xs[:, k, :] <- sum_s mix[s, k] xs[:, s, :] + b[k] y for all k at once, in place.  With ``a_next`` and ``w_next`` also
    returns rmsnorm(sum_k a_next[k] xs[:, k, :]) * w_next of the new streams (the next sublayer's operand)."""
    _need(xs, "xs", torch.float32)
    _need(y, "y", torch.float32)
    _need(mix, "mix", torch.float32)
    _need(b, "b", torch.float32)
    T, n, d = xs.shape
    if y.shape != (T, d) or mix.shape != (n, n) or b.numel() != n:
        raise KernelError("hyper_write: the sizes do not fit together")
    out = None
    if a_next is not None:
        _need(a_next, "a_next", torch.float32)
        _need(w_next, "w_next", torch.float32)
        if a_next.numel() != n or w_next.numel() != d:
            raise KernelError("hyper_write: the next read has the wrong sizes")
        out = torch.empty((T, d), dtype=out_dtype, device=xs.device)
    _work(f"hyper_write{' +read' if out is not None else ''} {T}x{n}x{d}", T * d * (8 * n + 4) + _nbytes(out))
    _check(lib().ik_hyper_write(_ptr(xs), _ptr(y), _ptr(mix), _ptr(b), _ptr(a_next), _ptr(w_next), _ptr(out),
                                _code(out) if out is not None else F32, T, n, d, eps, _stream()), "hyper_write")
    return out


def branch_norm_sum(ys, biases, weights, scales, out: torch.Tensor, eps: float, accumulate: bool) -> torch.Tensor:
    """out (+)= sum_b scales[b] * rmsnorm(ys[b] + biases[b]) * weights[b]: up to four float matrices [T, d]; a bias may be None."""
    n = len(ys)
    _need(out, "out", torch.float32)
    T, d = out.shape
    if not 1 <= n <= 4 or len(biases) != n or len(weights) != n or len(scales) != n:
        raise KernelError("branch_norm_sum: one to four branches, each with a weight and a constant")
    for y, bias, w in zip(ys, biases, weights):
        _need(y, "y", torch.float32)
        _need(w, "w", torch.float32)
        if y.shape != (T, d) or w.numel() != d or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != d)):
            raise KernelError("branch_norm_sum: the sizes do not fit together")
    arr = ctypes.c_void_p * n
    cs = (ctypes.c_float * n)(*[float(c) for c in scales])
    _work(f"branch_norm_sum {n}x{T}x{d}", (n + 1 + (1 if accumulate else 0)) * T * d * 4)
    _check(lib().ik_branch_norm_sum(arr(*[_ptr(y) for y in ys]), arr(*[_ptr(b) for b in biases]), arr(*[_ptr(w) for w in weights]),
                                    cs, n, _ptr(out), T, d, eps, 1 if accumulate else 0, _stream()), "branch_norm_sum")
    return out


def add_rows_(y: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """y[t, :] += v for every row of the float matrix ``y`` (a projection's bias)."""
    _need(y, "y", torch.float32)
    _need(v, "v", torch.float32)
    T, d = y.shape
    if v.numel() != d:
        raise KernelError("add_rows: the vector does not fit the rows")
    _work(f"add_rows {T}x{d}", 2 * _nbytes(y))
    _check(lib().ik_add_rows(_ptr(y), _ptr(v), T, d, _stream()), "add_rows")
    return y


def rmsnorm_range(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """RMS norm with a weight over ``x`` [rows, d], a column range of a wider float matrix (rows may lie further apart)."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(weight, "weight", torch.float32)
    rows, d = x.shape
    if x.stride(1) != 1 or weight.numel() != d:
        raise KernelError("rmsnorm_range: the sizes do not fit together")
    out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
    _work(f"rmsnorm_range {rows}x{d}", rows * d * (4 + out.element_size()))
    _check(lib().ik_rmsnorm_range(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), _code(out), rows, d, eps, _stream()), "rmsnorm_range")
    return out


# ---------------------------------------------------------------------------------------------
# Recurrences whose state decays row by row
DECAY_FORMS = {"softplus": 0, "double_exp": 1}


def decay_rows(x: torch.Tensor, bias: Optional[torch.Tensor], form: str, A_log: Optional[torch.Tensor] = None,
               per_head: int = 0) -> torch.Tensor:
    """Decays in (0, 1) from projections ``x`` [T, C] (float; a column range may be given).  ``softplus``:
    exp(-exp(A_log[c // per_head]) * softplus(x + bias)); ``double_exp``: exp(-exp(x + bias)).  Float arithmetic with the accurate exponential and logarithm."""
    _need(x, "x", torch.float32, contiguous=False)
    T, C = x.shape
    if x.stride(1) != 1 or (bias is not None and (bias.numel() != C or bias.dtype != torch.float32)):
        raise KernelError("decay_rows: the sizes do not fit together")
    if form == "softplus" and (A_log is None or per_head <= 0 or A_log.numel() * per_head != C):
        raise KernelError("decay_rows: the softplus form needs one A_log per head")
    out = torch.empty((T, C), dtype=torch.float32, device=x.device)
    _work(f"decay_rows {T}x{C}", 8 * T * C)
    _check(lib().ik_decay_rows(_ptr(x), x.stride(0), _ptr(bias), _ptr(A_log), _ptr(out), T, C, per_head, DECAY_FORMS[form], _stream()),
           "decay_rows")
    return out


def token_shift(x: torch.Tensor, mu: torch.Tensor, ring: torch.Tensor, ctx) -> torch.Tensor:
    """[n_mix, T, d]: x + (x' - x) * mu[m] with x' the input one position earlier in the same sequence (zeros at position
    0; across steps from ``ring`` [slots, 2, d] float, which then receives every sequence's last input)."""
    _need(x, "x")
    _need(mu, "mu", torch.float32)
    _need(ring, "ring", torch.float32)
    T, d = x.shape
    n_mix = mu.shape[0]
    if mu.shape != (n_mix, d) or tuple(ring.shape[1:]) != (2, d):
        raise KernelError("token_shift: the sizes do not fit together")
    out = torch.empty((n_mix, T, d), dtype=x.dtype, device=x.device)
    _work(f"token_shift {T}x{n_mix}x{d}", (n_mix + 2) * T * d * x.element_size())
    _check(lib().ik_token_shift(_ptr(x), _code(x), _ptr(mu), _ptr(ring), _ptr(ctx.slots), _ptr(ctx.cu_seqlens), _ptr(ctx.kv_lens),
                                _ptr(ctx.token_seq), _ptr(ctx.token_pos), _ptr(out), T * d, T, ctx.n_seqs, d, n_mix,
                                1 if ctx.is_decode else 0, _stream()), "token_shift", kernels=1 if ctx.is_decode else 2)
    return out


ROW_RULES = {"delta": 0, "bonus": 1}


def row_decay(rule: str, u: torch.Tensor, x1_off: int, k_off: int, v_off: int, dec: torch.Tensor, beta: Optional[torch.Tensor],
              bonus: Optional[torch.Tensor], state: torch.Tensor, ctx, n_heads: int, n_qk_heads: int, dk: int, dv: int) -> torch.Tensor:
    """A matrix state per head with a decay per key channel.  ``delta``: S <- diag(a) S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  ``bonus``: o = (S + diag(bonus) k v^T)^T r; S <- diag(w) S + k v^T.  q (or r), k and v are column ranges of
    the float matrix ``u``; ``dec`` [T, heads * dk]; ``beta`` [T, heads] (rows may lie further apart); ``bonus`` [heads * dk]; ``state`` [slots, 2, heads,
    dv, dk] float.  Returns [T, heads * dv] float."""
    _need(u, "u", torch.float32, contiguous=False)
    _need(dec, "dec", torch.float32)
    _need(state, "state", torch.float32)
    T = u.shape[0]
    H, G = n_heads, n_qk_heads
    if u.stride(1) != 1 or dec.shape != (T, H * dk) or tuple(state.shape[1:]) != (2, H, dv, dk) \
            or max(x1_off + G * dk, k_off + G * dk, v_off + H * dv) > u.shape[1] \
            or (rule == "delta" and (beta is None or beta.dtype != torch.float32 or beta.shape != (T, H) or beta.stride(1) != 1)) \
            or (rule == "bonus" and (bonus is None or bonus.dtype != torch.float32 or bonus.numel() != H * dk)):
        raise KernelError("row_decay: the sizes do not fit together")
    out = torch.empty((T, H * dv), dtype=torch.float32, device=u.device)
    n_state = ctx.n_seqs * H * dk * dv * 4
    _work(f"row_decay {rule} {T}x{H}x{dk}x{dv}", 2 * n_state + T * (2 * G * dk + H * dk + 2 * H * dv) * 4, 6 * T * H * dk * dv)
    st = lib().ik_row_decay(ROW_RULES[rule], _ptr(u), u.stride(0), x1_off, k_off, v_off, _ptr(dec), _ptr(beta), beta.stride(0) if beta is not None else 0, _ptr(bonus), _ptr(state),
                            _ptr(ctx.slots), _ptr(ctx.cu_seqlens), _ptr(ctx.kv_lens), _ptr(out), T, ctx.n_seqs, H, G, dk, dv,
                            1 if ctx.is_decode else 0, _stream())
    _check(st, "row_decay")
    return out
