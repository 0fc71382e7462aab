"""Python side of the CUDA kernels: thin wrappers that check shapes and dtypes, pass raw
device pointers and the current stream to the C entry points, and raise on any error.
Nothing here computes on the CPU or through a library: a missing build fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, found {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    """The tensor's address as ctypes takes it for a ``void*`` argument (an int, or None for a null pointer)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_device_index: Optional[int] = None


def set_device(index: Optional[int]) -> None:
    """The device whose current stream the kernels are launched on, when the caller knows it (an engine that
    lives on one device); None: ask torch for the current device at every call."""
    global _device_index
    _device_index = index


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current one), asked once per device."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = _device_index if _device_index is not None else torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


def _stream():
    """The current stream's handle. Every kernel call asks for it, so it comes from the one C call that
    returns the handle (torch.cuda.current_stream() builds a Python object around it at ten times the cost)."""
    if _raw_stream is not None:
        return _raw_stream(_device_index if _device_index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far in this process (graph replays are added by
    the code that replays them)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str, kernels: int = 1) -> None:
    global _launches
    if rc == 0:
        _launches += kernels
        return
    if rc == -2:
        raise KernelError(f"{what}: this size is outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {rc}")


_fn_cache = {}


def _fn(libname: str, symbol: str, argtypes):
    key = (libname, symbol)
    f = _fn_cache.get(key)
    if f is None:
        lib = build.load(libname)
        f = getattr(lib, symbol)
        f.argtypes = argtypes
        f.restype = _c_int
        _fn_cache[key] = f
    return f


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be contiguous int32")


# ---------------------------------------------------------------------------------------

def embedding_gather(tokens, table, out, status=None, scale: float = 1.0) -> None:
    """out[t,:] (fp32) = scale * table[tokens[t],:]."""
    _cuda(tokens, table, out, status)
    _i32(tokens, "tokens")
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous(),
          "embedding: out must be contiguous fp32, table contiguous")
    T, d = out.shape
    _need(table.shape[1] == d and tokens.numel() == T, "embedding: shape mismatch")
    f = _fn("embedding", "si_embedding_gather",
            [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p, _c_p])
    _check(f(_ptr(tokens), _ptr(table), _dt(table), _ptr(out), T, d, table.shape[0], float(scale),
             _ptr(status), _stream()), "embedding_gather")


# Most bytes that one launch fetches ahead into L2. Measured on the 8B shape: 4 to 8 MB, what arrives while
# the norm waits on its own loads, shortened a decode step by 0.5 to 1.3 % while only the norms triggered the
# launch of the kernel after them; now that the products do too, 0 to 8 MB differ by less than half a per cent
# either way (4 MB is never the worst), and 16 MB and more still lengthen the step.
AHEAD_BYTES = int(os.environ.get("SI_AHEAD_MB", "4")) << 20


def add_rmsnorm(resid, delta, weight, eps: float, out, rows=None, ahead=None, delta2=None) -> None:
    """resid (fp32, in place) += delta (+ delta2); out = weight * resid * rsqrt(mean(resid^2) + eps).

    With ``rows`` (int32 [R]) output row r comes from stream row rows[r] and resid stays
    as it is. ``ahead``: a tensor that the kernel after this one streams from memory (weights of
    the next matrix product); further blocks of this launch start fetching it into L2.
    """
    _cuda(resid, delta, weight, out, rows, delta2)
    _i32(rows, "rows")
    d = resid.shape[-1]
    if delta2 is not None:
        _need(delta is not None and delta2.dtype == out.dtype and delta2.is_contiguous() and delta2.shape == resid.shape,
              "add_rmsnorm: delta2 goes beside delta and must match resid's shape and out's dtype")
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous()
          and weight.is_contiguous(), "add_rmsnorm: tensors must be contiguous, resid fp32")
    _need(weight.numel() == d and out.shape[-1] == d, "add_rmsnorm: width mismatch")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == resid.shape,
              "add_rmsnorm: delta must match resid's shape and out's dtype")
    R = out.shape[0]
    _need(R == (rows.numel() if rows is not None else resid.shape[0]), "add_rmsnorm: row count mismatch")
    f = _fn("norm", "si_add_rmsnorm",
            [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p, _c_ll, _c_p])
    ahead_bytes = 0
    if ahead is not None:
        _cuda(ahead)
        ahead_bytes = min(ahead.numel() * ahead.element_size(), AHEAD_BYTES) if ahead.is_contiguous() else 0
    _check(f(_ptr(resid), _ptr(delta), _ptr(delta2), _ptr(rows), _ptr(weight), _dt(weight), _ptr(out), _dt(out),
             R, d, float(eps), _ptr(ahead) if ahead_bytes else None, ahead_bytes, _stream()), f"add_rmsnorm(hidden={d})")


def rmsnorm_rows(x, weight, eps: float, out=None) -> None:
    """out[..., :] = weight * x[..., :] * rsqrt(mean(x[..., :]^2) + eps) over the last dimension of a 2-D or 3-D
    tensor (or view: only the last dimension must be contiguous), in place by default. No residual stream is
    involved: for norms inside a part (a norm over each head of a stacked projection, say)."""
    out = x if out is None else out
    _cuda(x, weight, out)
    _need(x.dim() in (2, 3) and out.shape == x.shape and out.dtype == x.dtype, "rmsnorm_rows: x and out must be 2-D or 3-D and alike")
    _need(x.stride(-1) == 1 and out.stride(-1) == 1 and weight.is_contiguous() and weight.numel() == x.shape[-1],
          "rmsnorm_rows: the last dimension must be contiguous and as long as the weight")
    if x.dim() == 2:
        rows, inner = x.shape[0], 1
        xs, os_ = (x.stride(0), 0), (out.stride(0), 0)
    else:
        rows, inner = x.shape[0] * x.shape[1], x.shape[1]
        xs, os_ = (x.stride(0), x.stride(1)), (out.stride(0), out.stride(1))
    f = _fn("norm", "si_rmsnorm_rows", [_c_p, _c_p, _c_int, _c_p, _c_int, _c_ll, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll, _c_f, _c_p])
    _check(f(_ptr(x), _ptr(out), _dt(x), _ptr(weight), _dt(weight), rows, x.shape[-1], inner, xs[0], xs[1], os_[0], os_[1],
             float(eps), _stream()), f"rmsnorm_rows(n={x.shape[-1]})")


def add_norm(resid, delta=None, weight=None, eps: float = 0.0, out=None, rows=None, delta_weight=None,
             delta_eps: float = 0.0, delta_bias=None, extra=None, vec=None) -> None:
    """The residual add in its general form, all sums and statistics fp32:
        d = delta (+ delta_bias);  d <- delta_weight * d * rsqrt(mean(d^2) + delta_eps)  (with ``delta_weight``)
        resid (fp32, in place) += d (+ extra) (+ vec);   out = weight * resid * rsqrt(mean(resid^2) + eps)  (with ``out``)
    ``extra`` fp32 like resid, ``vec`` and ``delta_bias`` fp32 [hidden]. With ``rows`` (int32 [R]) output row r comes from
    stream row rows[r] and resid stays as it is."""
    _cuda(resid, delta, weight, out, rows, delta_weight, delta_bias, extra, vec)
    _i32(rows, "rows")
    d = resid.shape[-1]
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and resid.dim() == 2, "add_norm: resid must be contiguous fp32 rows")
    if out is not None:
        _need(weight is not None and weight.is_contiguous() and weight.numel() == d and out.is_contiguous()
              and out.shape[-1] == d, "add_norm: out needs a weight of the stream's width")
        _need(out.shape[0] == (rows.numel() if rows is not None else resid.shape[0]), "add_norm: row count mismatch")
    else:
        _need(rows is None, "add_norm: rows are for an output")
    xd = out if out is not None else delta
    if delta is not None:
        _need(delta.is_contiguous() and delta.shape == resid.shape and delta.dtype == xd.dtype,
              "add_norm: delta must match resid's shape and out's dtype")
    if delta_weight is not None:
        _need(delta is not None and delta_weight.is_contiguous() and delta_weight.numel() == d
              and (weight is None or weight.dtype == delta_weight.dtype), "add_norm: delta_weight must be like weight")
    _f32v(delta_bias, "delta_bias", d); _f32v(vec, "vec", d)
    if extra is not None:
        _need(extra.dtype == torch.float32 and extra.is_contiguous() and extra.shape == resid.shape, "add_norm: extra must be like resid")
    wd = weight if weight is not None else delta_weight
    R = out.shape[0] if out is not None else resid.shape[0]
    f = _fn("norm", "si_add_norm_general",
            [_c_p, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_ptr(resid), _ptr(delta), _ptr(delta_bias), _ptr(delta_weight), float(delta_eps), _ptr(extra), _ptr(vec),
             _ptr(rows), _ptr(weight), _dt(wd) if wd is not None else F32, _ptr(out), _dt(xd) if xd is not None else F32,
             R, d, float(eps), _stream()), f"add_norm(hidden={d})")


def rope_kv_write(qkv, positions, row_seq, inv_freq, rot_dim: int, block_table, k_cache, v_cache,
                  page_size: int, num_seqs: int, H: int, KV: int, hs: int, status=None) -> None:
    """Rotate q (in place) and k, store k and v of every row into its page.

    qkv: [T, (H+2KV)*hs]; k_cache/v_cache: [num_pages, KV, page_size, hs] of one layer, or None
    to rotate q only; inv_freq: fp32 [rot_dim/2] or None for no rotation.
    """
    _cuda(qkv, positions, row_seq, inv_freq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (H + 2 * KV) * hs, "rope_kv_write: qkv shape")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim,
              "rope_kv_write: inv_freq must be fp32 [rot_dim/2]")
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous(), "rope_kv_write: cache dtype/layout")
        _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.shape == v_cache.shape,
              "rope_kv_write: cache must be [pages, KV, page_size, hs]")
        num_pages = k_cache.shape[0]
    f = _fn("rope_kv", "si_rope_kv_write",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(qkv), _dt(qkv), qkv.stride(0), _ptr(positions), _ptr(row_seq), _ptr(inv_freq),
             rot_dim, _ptr(block_table), block_table.shape[1], _ptr(k_cache), _ptr(v_cache),
             num_pages, page_size, T, num_seqs, H, KV, hs, _ptr(status), _stream()),
           f"rope_kv_write(head_dim={hs}, rot_dim={rot_dim})")


def paged_attention_ref(q, k_cache, v_cache, block_table, row_seq, positions, out, page_size: int,
                        num_seqs: int, H: int, KV: int, hs: int, scale: float, window: int = 0,
                        status=None) -> None:
    """Plain fp32-arithmetic attention over the paged cache; q may be a strided row view."""
    _cuda(q, k_cache, v_cache, block_table, row_seq, positions, out, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = q.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * hs and out.shape[1] == H * hs,
          "paged_attention_ref: q/out shape")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "paged_attention_ref: dtypes differ")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "paged_attention_ref: cache must be [pages, KV, page_size, hs]")
    f = _fn("attention_ref", "si_paged_attention_ref",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
    _check(f(_ptr(q), _dt(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(row_seq), _ptr(positions), _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, T, num_seqs, H, KV, hs, float(scale), int(window or 0),
             _ptr(status), _stream()), f"paged_attention_ref(head_dim={hs})")


def swiglu(gu, out, group=None) -> None:
    """out[t,f] = silu(gate[t,f]) * up[t,f] from the stacked projection gu[t, 0..2F): gates and ups
    interleaved in groups of ``group`` columns (default F: all gates, then all ups)."""
    _cuda(gu, out)
    T, F = out.shape
    group = F if group is None else int(group)
    _need(gu.shape == (T, 2 * F) and gu.is_contiguous() and out.is_contiguous()
          and gu.dtype == out.dtype, "swiglu: gu must be [T, 2F] like out [T, F]")
    _need(group > 0 and F % group == 0, "swiglu: the group must divide F")
    f = _fn("swiglu", "si_swiglu", [_c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(gu), _ptr(out), _dt(out), T, F, group, _stream()), "swiglu")


def gemm_f32(a, w, out) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true fp32 (FFMA)."""
    _cuda(a, w, out)
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: fp32 tensors only")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1
          and out.stride(1) == 1, "gemm_f32: shapes/strides")
    f = _fn("gemm_f32", "si_gemm_f32",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K,
             _stream()), f"gemm_f32(M={M}, N={N}, K={K})")


def sample(logits, out, temperature=None, top_k=None, top_p=None, seed=None, counter=None) -> None:
    """Pick one token per row of fp32 logits; all per-row parameter tensors are optional
    (absent temperature means greedy)."""
    _cuda(logits, out, temperature, top_k, top_p, seed, counter)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be fp32 rows")
    _i32(out, "out"); _i32(top_k, "top_k")
    R, V = logits.shape
    for t, dt, nm in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                      (seed, torch.int64, "seed"), (counter, torch.int64, "counter")):
        if t is not None:
            _need(t.dtype == dt and t.numel() == R and t.is_contiguous(), f"sample: {nm} must be {dt} [rows]")
    f = _fn("sampling", "si_sample",
            [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
             _ptr(seed), _ptr(counter), _ptr(out), _stream()), "sample")


def argmax_scratch_words(rows: int) -> int:
    lib = build.load("sampling")
    lib.si_argmax_scratch_words.restype = _c_ll
    return int(lib.si_argmax_scratch_words(_c_int(rows)))


def argmax(logits, out, scratch) -> None:
    """Greedy pick per row of fp32 logits (ties to the lowest index) with the vocabulary of a row split over
    many blocks; ``scratch``: int32, ``argmax_scratch_words(capacity)`` long for some capacity >= rows,
    zeroed once by the caller and then left to this function."""
    _cuda(logits, out, scratch)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "argmax: logits must be fp32 rows")
    _i32(out, "out"); _i32(scratch, "scratch")
    R, V = logits.shape
    capacity = scratch.numel() // argmax_scratch_words(1)
    _need(capacity >= R and scratch.is_contiguous(), "argmax: scratch too small")
    f = _fn("sampling", "si_argmax", [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_int, _c_p, _c_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(scratch), capacity, _ptr(out), _stream()), "argmax")


def selftest_wait_runs_out(status, limit: int = 4096, gave_up=None) -> None:
    """Launch the self-test kernel whose bounded wait nothing ends: after ``limit`` probes it writes the
    wait-limit code into ``status`` (int32 [1]) and returns; ``gave_up`` (int32 [1], optional) is set to 1."""
    _cuda(status, gave_up)
    _i32(status, "status"); _i32(gave_up, "gave_up")
    f = _fn("selftest", "si_selftest_wait_runs_out", [_c_p, _c_int, _c_p, _c_p])
    _check(f(_ptr(status), int(limit), _ptr(gave_up), _stream()), f"selftest_wait_runs_out(limit={limit})")


# ---- tensor-core attention (bf16) ---------------------------------------------------------

_c_llr = ctypes.c_longlong


def attn_portion_tokens(H: int, KV: int, hs: int) -> int:
    """Most tokens of one item of the portion kernel (0: this head layout is not supported)."""
    lib = build.load("attention_mma")
    lib.si_attn_portion_tokens.restype = _c_int
    return lib.si_attn_portion_tokens(_c_int(H), _c_int(KV), _c_int(hs))


def attn_decode_rows(H: int, KV: int, hs: int) -> int:
    """Rows (tokens * heads per kv head) one item of the decode kernel may have; 0: none."""
    lib = build.load("attention_mma")
    lib.si_attn_decode_rows.restype = _c_int
    return lib.si_attn_decode_rows(_c_int(H), _c_int(KV), _c_int(hs))


def attn_decode_scratch_floats(num_items: int, H: int, KV: int, hs: int, nsplit: int) -> int:
    lib = build.load("attention_mma")
    lib.si_attn_decode_scratch_floats.restype = _c_llr
    return lib.si_attn_decode_scratch_floats(_c_int(num_items), _c_int(H), _c_int(KV), _c_int(hs), _c_int(nsplit))


def _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, what):
    _cuda(q, k_cache, v_cache, block_table, items, out)
    _i32(block_table, "block_table"); _i32(items, "items")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
          and v_cache.dtype == torch.bfloat16, f"{what}: bfloat16 tensors only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * hs and out.shape[1] == H * hs,
          f"{what}: q/out must be [T, H*hs] rows")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.is_contiguous() and v_cache.is_contiguous(),
          f"{what}: cache must be [pages, KV, page_size, hs]")
    _need(items.dim() == 2 and items.shape[1] == 4, f"{what}: items must be int32 [n, 4]")
    _need(q.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0,
          f"{what}: q and cache must be 16-byte aligned")


def attn_portion(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int,
                 KV: int, hs: int, scale: float, window: int = 0, status=None) -> None:
    """Tensor-core attention for prompt portions. ``items``: int32 [n, 4] rows
    (sequence, first row, tokens, first position), at most ``attn_portion_tokens`` tokens each."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_portion")
    f = _fn("attention_mma", "si_attn_portion",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(items), items.shape[0], _ptr(out), out.stride(0), k_cache.shape[0], page_size, num_seqs,
             H, KV, hs, float(scale), int(window or 0), _ptr(status), _stream()),
           f"attn_portion(heads={H}, kv_heads={KV}, head_dim={hs})")


def attn_decode(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int, KV: int,
                hs: int, scale: float, window: int = 0, nsplit: int = 1, scratch=None, status=None) -> None:
    """Tensor-core attention for decode rows and short portions (at most
    ``attn_decode_rows // (H // KV)`` tokens an item). With ``nsplit`` > 1 the key range is split
    over blocks and ``scratch`` (fp32, ``attn_decode_scratch_floats`` elements, zero before its
    first use) holds the partials and the tickets of the merge."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_decode")
    if nsplit > 1:
        _cuda(scratch)
        need = attn_decode_scratch_floats(items.shape[0], H, KV, hs, nsplit)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode: scratch must hold {need} floats")
    f = _fn("attention_mma", "si_attn_decode",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(items), items.shape[0], _ptr(out), out.stride(0), k_cache.shape[0], page_size, num_seqs,
             H, KV, hs, float(scale), int(window or 0), int(nsplit), _ptr(scratch), _ptr(status), _stream()),
           f"attn_decode(heads={H}, kv_heads={KV}, head_dim={hs})")


# ---- decode attention with TMA-fed tiles ----------------------------------------------------

MAX_KEPT_MAPS = 4096      # descriptors kept per table; the oldest goes when a new one would exceed it


def _keep_map(table: dict, key, ent) -> None:
    """Descriptors are kept by (device, address, shape): a tensor at the same place with the same shape has
    the same descriptor, so an entry that outlives its tensor is still right for the next one there. The
    table is bounded, so that a process that builds engine after engine does not grow it for ever."""
    while len(table) >= MAX_KEPT_MAPS:
        table.pop(next(iter(table)))
    table[key] = ent


_tensor_maps = {}


def attn_decode_tma_ok(H: int, KV: int, hs: int, page_size: int) -> bool:
    """True when the TMA decode kernel takes this head layout and page size."""
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_ok.restype = _c_int
    return bool(lib.si_attn_decode_tma_ok(_c_int(H), _c_int(KV), _c_int(hs), _c_int(page_size)))


def attn_decode_tma_rows(H: int, KV: int) -> int:
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_rows.restype = _c_int
    return lib.si_attn_decode_tma_rows(_c_int(H), _c_int(KV))


def attn_decode_tma_scratch_floats(num_items: int, H: int, KV: int, hs: int, nsplit: int) -> int:
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_scratch_floats.restype = _c_llr
    return lib.si_attn_decode_tma_scratch_floats(_c_int(num_items), _c_int(H), _c_int(KV), _c_int(hs), _c_int(nsplit))


def _cache_map(cache: torch.Tensor):
    """The TMA descriptor of one layer's K or V cache; made once per tensor and kept."""
    key = (cache.device.index, cache.data_ptr(), tuple(cache.shape))
    ent = _tensor_maps.get(key)
    if ent is None:
        raw = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(raw) + 63) & ~63
        num_pages, KV, page_size, hs = cache.shape
        f = _fn("attention_tma", "si_attn_encode_cache_map", [_c_p, _c_p, _c_ll, _c_int, _c_int, _c_int])
        rc = f(_c_p(addr), _ptr(cache), num_pages, KV, page_size, hs)
        if rc != 0:
            raise KernelError(f"cannot describe the cache {tuple(cache.shape)} to the TMA unit (code {rc})")
        ent = (raw, addr)
        _keep_map(_tensor_maps, key, ent)
    return _c_p(ent[1])


def split_work(tiles, budget: int, entries: int, max_splits: int = 128, min_tiles: int = 1):
    """Cut decode items into shares of about equal length. ``tiles[i]``: 64-key tiles that item i reads
    (0: an empty item, which gets no entry). ``budget``: shares that run at the same time. With no more
    items than that, the shares are as short as ``budget`` shares in all allow (the smallest length L with
    sum(ceil(tiles / L)) <= budget): more would run in a second round, fewer would leave the longest item
    to few blocks. With more items than that the cut is chosen by an estimate of the time (see the code), so
    that a long item among many short ones is still cut and the last blocks do not run alone. No share is shorter than ``min_tiles``, no item has more than ``max_splits``. Returns
    an int32 array [entries, 4] of (item, split, splits of the item, first slot of the item), longest
    shares first, the rest filled with item -1: ``attn_decode_tma(work=...)``. ``entries >= budget +
    len(tiles)`` always suffices; more entries allow finer cuts when items outnumber the budget."""
    import numpy as np
    key = (tuple(tiles), budget, entries, max_splits, min_tiles)
    if _split_memo.get("key") == key:               # tile counts change once in 64 decode steps of a sequence
        return _split_memo["work"]
    _split_memo["key"], _split_memo["work"] = key, _split_work(np, tiles, budget, entries, max_splits, min_tiles)
    return _split_memo["work"]


_split_memo: dict = {}


def _split_work(np, tiles, budget, entries, max_splits, min_tiles):
    t = np.asarray(tiles, dtype=np.int64)
    live = np.flatnonzero(t > 0)
    out = np.full((entries, 4), -1, dtype=np.int32)
    out[:, 1:] = 0
    if live.size == 0:
        return out
    tl = t[live]

    def splits_for(L):
        return np.minimum(max_splits, -(-tl // max(L, min_tiles, 1)))

    if live.size <= budget:
        lo, hi = 1, int(tl.max())                    # smallest L whose shares fit the budget
        while lo < hi:
            mid = (lo + hi) // 2
            if int(splits_for(mid).sum()) <= budget:
                hi = mid
            else:
                lo = mid + 1
        sp = splits_for(lo)
    else:
        # More items than shares that run at once. Blocks follow one another on the block slots; what counts is
        # the longest chain on a slot (about ceil(shares / slots) shares of length L, at most load / slots + L),
        # the time HBM needs for everything (reached with about four fifths of the slots busy), and what a
        # share costs beside its tiles (about eight tiles' time for a full round of them: start, partial
        # results, merge). The cut with the least of these wins among 1 to 32 cuts of the longest item, as far
        # as the entries reach: many equal sequences stay whole, a few more sequences than slots are cut in
        # four or five so that the last blocks do not run alone, a long one among many short ones is cut most.
        load, slots, tmax = float(tl.sum()), float(max(budget, 1)), int(tl.max())
        best = None
        for k in (1, 2, 3, 4, 5, 6, 8, 12, 16, 32):
            L = max(-(-tmax // k), min_tiles, 1)
            cand = splits_for(L)
            n = int(cand.sum())
            if n > entries and best is not None:
                break
            longest = int((-(-tl // cand)).max())
            chain = min(-(-n // int(slots)) * longest, load / slots + longest)
            cost = max(chain, load / (0.8 * slots)) + 8.0 * n / slots
            if best is None or cost < best[0]:
                best = (cost, cand)
            if L <= max(min_tiles, 1):
                break
        sp = best[1]
    if int(sp.sum()) > entries:
        raise ValueError(f"split_work: {int(sp.sum())} shares do not fit {entries} entries")
    first = np.cumsum(sp) - sp
    order = np.argsort(-(-(-tl // sp)), kind="stable")          # longest shares first: they start first
    so = sp[order]
    total = int(so.sum())
    out[:total, 0] = np.repeat(live[order], so)
    out[:total, 1] = np.arange(total) - np.repeat(np.cumsum(so) - so, so)
    out[:total, 2] = np.repeat(so, so)
    out[:total, 3] = np.repeat(first[order], so)
    return out


_work_floats_memo: dict = {}


def attn_decode_tma_work_floats(slots: int, H: int, KV: int, hs: int) -> int:
    key = (slots, H, KV, hs)
    n = _work_floats_memo.get(key)
    if n is None:
        lib = build.load("attention_tma")
        lib.si_attn_decode_tma_work_floats.restype = _c_llr
        n = _work_floats_memo[key] = lib.si_attn_decode_tma_work_floats(_c_int(slots), _c_int(H), _c_int(KV), _c_int(hs))
    return n


def attn_decode_tma(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int, KV: int,
                    hs: int, scale: float, window: int = 0, nsplit: int = 1, scratch=None, status=None,
                    max_rows: int = 0, work=None) -> None:
    """``attn_decode`` with the K/V tiles fetched by TMA (head_dim 64 or 128, page sizes 8 to 64);
    items hold at most ``attn_decode_tma_rows // (H // KV)`` tokens. ``max_rows``: the most rows
    (tokens x query heads of a KV head) of any item when the caller knows it (0: unknown); at most 8
    rows run the variant with the products taken the other way round.
    ``work`` (int32 [W, 4], rows of (item, split, splits of that item, first slot of that item); item -1:
    nothing): every item is cut into its own number of shares, ``nsplit`` is not used, and ``scratch``
    holds ``attn_decode_tma_work_floats(W, ...)`` floats. Made by ``split_work``."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_decode_tma")
    if work is not None:
        _cuda(work, scratch)
        _need(work.dtype == torch.int32 and work.dim() == 2 and work.shape[1] == 4 and work.is_contiguous(),
              "attn_decode_tma: work must be int32 [W, 4]")
        need = attn_decode_tma_work_floats(work.shape[0], H, KV, hs)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode_tma: scratch must hold {need} floats")
    elif nsplit > 1:
        _cuda(scratch)
        need = attn_decode_tma_scratch_floats(items.shape[0], H, KV, hs, nsplit)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode_tma: scratch must hold {need} floats")
    f = _fn("attention_tma", "si_attn_decode_tma",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_int, _c_int, _c_p, _c_int, _c_p, _c_p])
    W = work.shape[0] if work is not None else 0
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _cache_map(k_cache), _cache_map(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(items), items.shape[0], _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, num_seqs, H, KV, hs, float(scale), int(window or 0), int(nsplit),
             _ptr(work), W, W, _ptr(scratch), int(max_rows), _ptr(status), _stream()),
           f"attn_decode_tma(heads={H}, kv_heads={KV}, head_dim={hs}, page_size={page_size})")


# ---- few-row matrix product (decode) ----------------------------------------------------------

SKINNY_MAX_ROWS = 16


def gemm_skinny_ok(a, w, out) -> bool:
    """True when the few-row kernel takes these tensors (bf16, at most 16 rows, K a multiple of 8)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and out.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a, w, out, checked: bool = False) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T for M <= 16: the weights stream through mma.sync fragments.
    ``checked``: the caller has just asked ``gemm_skinny_ok`` for these tensors."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_skinny: shapes")
    _need(checked or gemm_skinny_ok(a, w, out),
          "gemm_skinny: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_skinny", "si_gemm_skinny",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _dt(out), M, N, K, _stream()),
           f"gemm_skinny(M={M}, N={N}, K={K})")


def gemm_skinny_batched(a, w, out) -> None:
    """out[b] = a[b] @ w[b]^T for every b in one launch: ``a`` [B, M, K], ``w`` [B, N, K], ``out`` [B, M, N], M <= 16; each
    product must be one that ``gemm_skinny`` takes (the caller has asked ``gemm_skinny_ok`` for one of them), and the
    strides between products multiples of 8 entries."""
    _cuda(a, w, out)
    B, M, K = a.shape
    N = w.shape[1]
    _need(w.shape == (B, N, K) and out.shape == (B, M, N) and a.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1,
          "gemm_skinny_batched: shapes")
    _need(gemm_skinny_ok(a[0], w[0], out[0]) and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0,
          "gemm_skinny_batched: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows and products")
    f = _fn("gemm_skinny", "si_gemm_skinny_batched",
            [_c_p, _c_ll, _c_ll, _c_p, _c_ll, _c_ll, _c_p, _c_ll, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(1), a.stride(0), _ptr(w), w.stride(1), w.stride(0), _ptr(out), out.stride(1), out.stride(0),
             _dt(out), B, M, N, K, _stream()), f"gemm_skinny_batched(B={B}, M={M}, N={N}, K={K})")


def gemm_skinny_relu2(a, w, out, checked: bool = False) -> None:
    """out[M,N] (bf16) = relu(a[M,K] @ w[N,K]^T)^2 for M <= 16: the activation runs in the product's epilogue."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N) and out.dtype == torch.bfloat16, "gemm_skinny_relu2: shapes, bf16 output")
    _need(checked or gemm_skinny_ok(a, w, out), "gemm_skinny_relu2: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_skinny", "si_gemm_skinny_relu2", [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()),
           f"gemm_skinny_relu2(M={M}, N={N}, K={K})")


def gemm_skinny_swiglu(a, w, out, checked: bool = False) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T for M <= 16, the rows of w interleaved in groups of 8
    (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_skinny_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(checked or gemm_skinny_ok(a, w, out), "gemm_skinny_swiglu: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_skinny", "si_gemm_skinny_swiglu", [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, F, K, _stream()),
           f"gemm_skinny_swiglu(M={M}, F={F}, K={K})")


def gemm_skinny_glu_limited(a, w, bias, out, limit: float, alpha: float, checked: bool = False) -> None:
    """out[M,F] = g * sigmoid(alpha g) * (u + 1), g = min(gate + bias, limit), u = clamp(up + bias, -limit, limit), of
    a[M,K] @ w[2F,K]^T for M <= 16, the rows of w (and the entries of ``bias``, fp32 [2F] or None) interleaved in groups of
    8: the activation runs in the product's epilogue."""
    _cuda(a, w, bias, out)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_skinny_glu_limited: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(checked or gemm_skinny_ok(a, w, out), "gemm_skinny_glu_limited: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    _f32v(bias, "bias", 2 * F)
    f = _fn("gemm_skinny", "si_gemm_skinny_glu_limited",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_f, _c_f, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, F, K, _ptr(bias), float(limit), float(alpha),
             _stream()), f"gemm_skinny_glu_limited(M={M}, F={F}, K={K})")


def gemm_skinny_qkv_rope(a, w, out, positions, row_seq, inv_freq, block_table, k_cache, v_cache, page_size: int,
                         num_seqs: int, H: int, KV: int, hs: int, status=None) -> None:
    """The stacked q/k/v projection of at most 16 rows with what ``rope_kv_write`` would do next in its epilogue:
    q and k heads rotated by their row's position (the whole head, rotate-half pairs), q written to
    ``out[:, :H*hs]``, k and v stored into the rows' cache pages (``k_cache`` None: nothing stored). The k and v
    columns of ``out`` are left as they are."""
    _cuda(a, w, out, positions, row_seq, inv_freq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    M, K = a.shape
    _need(w.shape == ((H + 2 * KV) * hs, K) and out.shape[0] == M and out.shape[1] >= H * hs and out.dtype == torch.bfloat16,
          "gemm_skinny_qkv_rope: w must be [(H + 2 KV) * hs, K], out [M, >= H * hs] bf16")
    _need(gemm_skinny_ok(a, w, out) and hs % 16 == 0, "gemm_skinny_qkv_rope: bf16 inputs, at most 16 rows, K a multiple of 8, "
          "16-byte aligned rows, head_dim a multiple of 16")
    _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == hs,
          "gemm_skinny_qkv_rope: inv_freq must be fp32 [head_dim / 2] (the whole head is rotated)")
    _need(positions.numel() == M and row_seq.numel() == M, "gemm_skinny_qkv_rope: one position and sequence per row")
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k_cache.is_contiguous()
              and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (KV, page_size, hs)
              and k_cache.shape == v_cache.shape, "gemm_skinny_qkv_rope: cache must be bf16 [pages, KV, page_size, hs]")
        num_pages = k_cache.shape[0]
    f = _fn("gemm_skinny", "si_gemm_skinny_qkv_rope",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, K, _ptr(positions), _ptr(row_seq),
             _ptr(inv_freq), _ptr(block_table), block_table.shape[1] if block_table is not None else 0, _ptr(k_cache),
             _ptr(v_cache), num_pages, page_size, num_seqs, H, KV, hs, _ptr(status), _stream()),
           f"gemm_skinny_qkv_rope(M={M}, heads={H}, kv_heads={KV}, head_dim={hs})")


# ---- tcgen05 matrix product (many rows) -------------------------------------------------------

_weight_maps = {}


_tc05_available = None


def gemm_tc05_available() -> bool:
    """True when the driver hands out the tensor-map encoder that the TMA-fed kernels need."""
    global _tc05_available
    if _tc05_available is None:
        lib = build.load("gemm_tc05")
        lib.si_gemm_tc05_ok.restype = _c_int
        _tc05_available = bool(lib.si_gemm_tc05_ok())
    return _tc05_available


def gemm_tc05_ok(a, w, out) -> bool:
    """True when the tcgen05 kernel takes these tensors (bf16, K a multiple of 8, aligned rows)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _weight_map(w: torch.Tensor, box_rows: int = 256):
    """The weight's TMA descriptor with boxes of ``box_rows`` rows (256: one CTA a tile; 128: a pair of CTAs)."""
    key = (w.device.index, w.data_ptr(), tuple(w.shape), w.stride(0), box_rows)
    ent = _weight_maps.get(key)
    if ent is None:
        raw = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(raw) + 63) & ~63
        f = _fn("gemm_tc05", "si_gemm_tc05_encode_weight", [_c_p, _c_p, _c_int, _c_int, _c_ll, _c_int])
        rc = f(_c_p(addr), _ptr(w), w.shape[0], w.shape[1], w.stride(0), box_rows)
        if rc != 0:
            raise KernelError(f"cannot describe the weight {tuple(w.shape)} to the TMA unit (code {rc})")
        ent = (raw, addr)
        _keep_map(_weight_maps, key, ent)
    return _c_p(ent[1])


def gemm_tc05(a, w, out, status=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory)."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_tc05: shapes")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None          # more than one tile of rows: pairs of CTAs take tiles together
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), _dt(out), M, N, K, _ptr(status),
             _stream()), f"gemm_tc05(M={M}, N={N}, K={K})")


def gemm_tc05_add(a, w, resid, status=None) -> None:
    """resid[M,N] (fp32) += a[M,K] @ w[N,K]^T on the tcgen05 tensor cores, each sum rounded to bf16 before the add
    (what storing the product in bf16 and adding it in the norm kernel gives)."""
    _cuda(a, w, resid, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and resid.shape == (M, N) and resid.dtype == torch.float32 and resid.stride(1) == 1,
          "gemm_tc05_add: resid must be fp32 [M, N] rows")
    _need(gemm_tc05_ok(a, w, resid), "gemm_tc05_add: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_add", [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(resid), resid.stride(0), M, N, K, _ptr(status), _stream()),
           f"gemm_tc05_add(M={M}, N={N}, K={K})")


def gemm_tc05_glu_limited(a, w, bias, out, limit: float, alpha: float, status=None) -> None:
    """``gemm_skinny_glu_limited`` for many rows, on the tcgen05 tensor cores."""
    _cuda(a, w, bias, out, status)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16 and out.stride(1) == 1,
          "gemm_tc05_glu_limited: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05_glu_limited: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    _f32v(bias, "bias", 2 * F)
    f = _fn("gemm_tc05", "si_gemm_tc05_glu_limited",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_f, _c_f, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), M, F, K, _ptr(bias), float(limit), float(alpha),
             _ptr(status), _stream()), f"gemm_tc05_glu_limited(M={M}, F={F}, K={K})")


def gemm_tc05_relu2(a, w, out, status=None) -> None:
    """out[M,N] (bf16) = relu(a[M,K] @ w[N,K]^T)^2 on the tcgen05 tensor cores, the activation in the epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N) and out.dtype == torch.bfloat16, "gemm_tc05_relu2: shapes, bf16 output")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05_relu2: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_relu2", [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), M, N, K, _ptr(status), _stream()),
           f"gemm_tc05_relu2(M={M}, N={N}, K={K})")


def gemm_tc05_swiglu(a, w, out, status=None) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T on the tcgen05 tensor cores, the rows of w interleaved
    in groups of 8 (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_tc05_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05_swiglu: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_swiglu", [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), M, F, K, _ptr(status), _stream()),
           f"gemm_tc05_swiglu(M={M}, F={F}, K={K})")


# ---- tcgen05 matrix product for up to 128 rows ------------------------------------------------------

ROWS_MAX = 128


def gemm_rows_ok(a, w, out) -> bool:
    """True when the product for up to 128 rows takes these tensors (bf16, K a multiple of 8, aligned rows)."""
    return a.shape[0] <= ROWS_MAX and gemm_tc05_ok(a, w, out)


def gemm_rows(a, w, out, status=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T for M <= 128 on the tcgen05 tensor cores: a tile of 128 output columns a
    block, the k range of a tile cut over a cluster where the tiles alone do not fill the GPU (see gemm_rows.cu)."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_rows: shapes")
    _need(gemm_rows_ok(a, w, out), "gemm_rows: bf16 inputs, at most 128 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_rows", "si_gemm_rows", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _weight_map(w, 128), _ptr(out), out.stride(0), _dt(out), M, N, K,
             _ptr(status), _stream()), f"gemm_rows(M={M}, N={N}, K={K})")


def gemm_rows_swiglu(a, w, out, status=None) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T for M <= 128, the rows of w interleaved in groups of 8
    (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_rows_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(gemm_rows_ok(a, w, out), "gemm_rows_swiglu: bf16 inputs, at most 128 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_rows", "si_gemm_rows_swiglu", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _weight_map(w, 128), _ptr(out), out.stride(0), M, F, K,
             _ptr(status), _stream()), f"gemm_rows_swiglu(M={M}, F={F}, K={K})")


# ---- prompt-portion attention on tcgen05 ---------------------------------------------------------

def attn_portion_tc05_ok(H: int, KV: int, hs: int, page_size: int) -> bool:
    lib = build.load("attention_tc05")
    lib.si_attn_portion_tc05_ok.restype = _c_int
    return bool(lib.si_attn_portion_tc05_ok(_c_int(H), _c_int(KV), _c_int(hs), _c_int(page_size)))


def attn_portion_tc05_tokens(H: int, KV: int) -> int:
    """Most tokens of one work item of ``attn_portion_tc05``."""
    lib = build.load("attention_tc05")
    lib.si_attn_portion_tc05_tokens.restype = _c_int
    return lib.si_attn_portion_tc05_tokens(_c_int(H), _c_int(KV))


def attn_portion_tc05(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int,
                      KV: int, hs: int, scale: float, window: int = 0, status=None, slopes=None, q_temp=None, gate=None) -> None:
    """``attn_portion`` on the tcgen05 tensor cores (TMA-fed K/V tiles, S and P V in tensor memory);
    head_dim 64 or 128, page sizes 8 to 64, items of at most ``attn_portion_tc05_tokens`` tokens. ``v_cache`` None: the
    values are the keys. ``slopes``, ``q_temp`` (a coefficient that is not negative) and ``gate`` as in ``attention_general``
    (the gate's rows 16-byte aligned)."""
    if v_cache is None:
        v_cache = k_cache
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_portion_tc05")
    _cuda(slopes, gate)
    _f32v(slopes, "slopes", H)
    qt_coef, qt_every = _q_temp(q_temp)
    _need(qt_coef >= 0.0, "attn_portion_tc05: a query temperature with a negative coefficient is not supported")
    _need(gate is None or (gate.dtype == torch.bfloat16 and gate.shape == (q.shape[0], H * hs) and gate.stride(1) == 1
                           and gate.stride(0) % 8 == 0 and gate.data_ptr() % 16 == 0), "attn_portion_tc05: gate must be bf16 [T, H*hs], rows 16-byte aligned")
    f = _fn("attention_tc05", "si_attn_portion_tc05",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_f, _c_int, _c_p, _c_ll, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _cache_map(k_cache), _cache_map(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(items), items.shape[0], _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, num_seqs, H, KV, hs, float(scale), int(window or 0), _ptr(slopes), qt_coef, qt_every,
             _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(status),
             _stream()), f"attn_portion_tc05(heads={H}, kv_heads={KV}, head_dim={hs}, page_size={page_size})")


# ---- general attention, stores, latent form -------------------------------------------------------

def embedding_pair(tokens, positions, row_seq, q_start, slots, last_token, table, pair, out, buckets: int,
                   mul_prev: int, mul_cur: int, num_seqs: int, status=None) -> None:
    """out[t,:] (fp32) = table[tokens[t],:] + pair[r_t,:], r_t = (previous token * mul_prev + token * mul_cur) mod
    buckets, r = buckets for a sequence's first token. ``last_token`` (int32 [slots]) holds every request's latest
    token between steps; the kernel reads and renews it."""
    _cuda(tokens, positions, row_seq, q_start, slots, last_token, table, pair, out, status)
    for t, nm in ((tokens, "tokens"), (positions, "positions"), (row_seq, "row_seq"), (q_start, "q_start"),
                  (slots, "slots"), (last_token, "last_token")):
        _i32(t, nm)
    T, d = out.shape
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and pair.is_contiguous()
          and table.dtype == pair.dtype, "embedding_pair: out must be contiguous fp32, tables contiguous and alike")
    _need(table.shape[1] == d and pair.shape == (buckets + 1, d) and tokens.numel() == T,
          "embedding_pair: shape mismatch (the pair table has buckets + 1 rows)")
    f = _fn("embedding", "si_embedding_pair",
            [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll,
             _c_int, _c_p, _c_p])
    _check(f(_ptr(tokens), _ptr(positions), _ptr(row_seq), _ptr(q_start), _ptr(slots), _ptr(last_token), _ptr(table),
             _ptr(pair), _dt(table), _ptr(out), T, d, table.shape[0], int(buckets), int(mul_prev), int(mul_cur),
             int(num_seqs), _ptr(status), _stream()), "embedding_pair")


def _f32v(t, name: str, n=None) -> None:
    if t is not None:
        _need(t.dtype == torch.float32 and t.is_contiguous() and (n is None or t.numel() == n),
              f"{name} must be contiguous fp32" + (f" of {n} elements" if n is not None else ""))


def _q_temp(q_temp):
    """(coef, every) of a query temperature as the kernels take it; None: (0, 0), no temperature."""
    if q_temp is None:
        return 0.0, 0
    coef, every = float(q_temp[0]), int(q_temp[1])
    _need(every > 0 and every == q_temp[1], "query temperature: 'every' must be a positive whole number")
    return coef, every


def attention_general(q, k_cache, v_cache, block_table, row_seq, positions, out, page_size: int, num_seqs: int,
                      H: int, KV: int, dk: int, dv: int, scale: float, window: int = 0, dist_bias=None, sink=None,
                      status=None, softcap: float = 0.0, v_share: int = 1, slopes=None, q_temp=None, gate=None) -> None:
    """fp32-arithmetic attention over the paged cache with key size ``dk``, value size ``dv``, values from
    ``v_cache`` or (None) the first ``dv`` entries of the keys, a bias by distance ``dist_bias`` (fp32 [nd, H],
    row min(distance, nd - 1)) and a sink per head (fp32 [H]) in the softmax denominator. ``softcap`` > 0: the scaled
    score s becomes softcap * tanh(s / softcap). ``v_share`` > 1: that many neighbouring key heads read one value head
    (``v_cache`` holds KV / v_share heads). ``slopes`` (fp32 [H]): ``slopes[h] * (i - j)`` is taken off the scaled score of
    query i and key j. ``q_temp`` ``(coef, every)``: row i's scale is multiplied by 1 + coef * ln(floor((i + 1) / every) + 1).
    ``gate`` ([T, H*dv] like ``q``, rows with a stride): the result is multiplied entry by entry with sigmoid(gate).
    ``out`` may be fp32 whatever the storage."""
    _cuda(q, k_cache, v_cache, block_table, row_seq, positions, out, dist_bias, sink, slopes, gate, status)
    _need(gate is None or (gate.dtype == q.dtype and gate.shape == (q.shape[0], H * dv) and gate.stride(1) == 1),
          "attention_general: gate must be [T, H*dv] in q's dtype")
    _f32v(slopes, "slopes", H)
    qt_coef, qt_every = _q_temp(q_temp)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = q.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * dk and out.shape[1] == H * dv,
          "attention_general: q must be [T, H*dk], out [T, H*dv]")
    _need(q.dtype == k_cache.dtype and out.dtype in (q.dtype, torch.float32)
          and (v_cache is None or v_cache.dtype == q.dtype), "attention_general: dtypes differ")
    _need(v_share >= 1 and KV % v_share == 0 and (v_share == 1 or v_cache is not None), "attention_general: v_share")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, dk) and k_cache.is_contiguous(),
          "attention_general: keys must be [pages, KV, page_size, dk]")
    if v_cache is not None:
        _need(tuple(v_cache.shape) == (k_cache.shape[0], KV // v_share, page_size, dv) and v_cache.is_contiguous(),
              "attention_general: values must be [pages, KV / v_share, page_size, dv]")
    nd = 0
    if dist_bias is not None:
        _need(dist_bias.dim() == 2 and dist_bias.shape[1] == H, "attention_general: dist_bias must be [nd, H]")
        _f32v(dist_bias, "dist_bias")
        nd = dist_bias.shape[0]
    _f32v(sink, "sink", H)
    f = _fn("attention_general", "si_attention_general",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_int, _c_p, _c_f, _c_int, _c_int, _c_p, _c_f, _c_int,
             _c_p, _c_ll, _c_p, _c_p])
    _check(f(_ptr(q), _dt(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(row_seq), _ptr(positions), _ptr(out), out.stride(0), k_cache.shape[0], page_size, T, num_seqs,
             H, KV, dk, dv, float(scale), int(window or 0), _ptr(dist_bias), nd, _ptr(sink), float(softcap or 0.0),
             int(v_share), 1 if out.dtype == torch.float32 and q.dtype != torch.float32 else 0, _ptr(slopes), qt_coef,
             qt_every, _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(status), _stream()),
           f"attention_general(dk={dk}, dv={dv})")


def kv_store(qkv, positions, row_seq, block_table, k_cache, v_cache, page_size: int, num_seqs: int, H: int,
             KV: int, dk: int, dv: int, status=None) -> None:
    """Rows [q: H*dk | k: KV*dk | v: KV*dv | ...]: k and v of every row into its page, unrotated. ``v_cache`` None with
    ``dv`` 0: the keys alone (a layer whose keys serve as its values)."""
    _cuda(qkv, positions, row_seq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= H * dk + KV * (dk + dv), "kv_store: row layout")
    _need(k_cache.dtype == qkv.dtype and k_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (KV, page_size, dk),
          "kv_store: keys must be [pages, KV, page_size, dk]")
    if v_cache is None:
        _need(dv == 0, "kv_store: without a value cache dv must be 0")
    else:
        _need(v_cache.dtype == qkv.dtype and v_cache.is_contiguous() and tuple(v_cache.shape) == (k_cache.shape[0], KV, page_size, dv),
              "kv_store: values must be [pages, KV, page_size, dv]")
    f = _fn("attention_general", "si_kv_store",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(qkv), _dt(qkv), qkv.stride(0), _ptr(positions), _ptr(row_seq), _ptr(block_table), block_table.shape[1],
             _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], page_size, qkv.shape[0], num_seqs, H, KV, dk, dv,
             _ptr(status), _stream()), f"kv_store(dk={dk}, dv={dv})")


def latent_prepare(kv, q, q_full, norm_w, eps: float, inv_freq, rot_dims: int, positions, row_seq, block_table,
                   k_cache, page_size: int, num_seqs: int, H: int, dq: int, dr: int, rk: int, status=None, q_exp=None,
                   interleaved: bool = False, rot_scale: float = 1.0) -> None:
    """The latent attention's step between its projections and the attention itself. ``kv`` [T, rk + dr]: the
    latent is normalised (weight ``norm_w``) and stored with the rotated shared key part as one key of rk + dr
    entries (``k_cache`` [pages, 1, page_size, rk + dr]; None: nothing stored). ``q`` [T, H * (dq + dr)]: every head's
    last dr entries are rotated into ``q_full[:, h, rk:]`` (``q_full`` [T, H * (rk + dr)]; its first rk entries per
    head are the caller's). The first ``rot_dims`` of the dr entries are rotated, in pairs (i, i + rot_dims/2) or, when
    ``interleaved``, (2i, 2i + 1); cosines and sines are multiplied by ``rot_scale``. ``q_exp`` (optional, like ``q``)
    receives every head's [plain part | rotated part]."""
    _cuda(kv, q, q_full, norm_w, inv_freq, positions, row_seq, block_table, k_cache, status, q_exp)
    if q_exp is not None:
        _need(q_exp.shape == q.shape and q_exp.dtype == q.dtype and q_exp.stride(1) == 1, "latent_prepare: q_exp must be like q")
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = kv.shape[0]
    _need(kv.stride(1) == 1 and q.stride(1) == 1 and q_full.stride(1) == 1 and kv.shape[1] == rk + dr
          and q.shape == (T, H * (dq + dr)) and q_full.shape == (T, H * (rk + dr)), "latent_prepare: shapes")
    _need(kv.dtype == q.dtype == q_full.dtype, "latent_prepare: dtypes differ")
    _f32v(norm_w, "norm_w", rk)
    _f32v(inv_freq, "inv_freq", rot_dims // 2)
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == kv.dtype and k_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (1, page_size, rk + dr),
              "latent_prepare: the cache must be [pages, 1, page_size, rk + dr]")
        num_pages = k_cache.shape[0]
    f = _fn("attention_general", "si_latent_prepare",
            [_c_p, _c_int, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_f, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_p,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_p, _c_p])
    _check(f(_ptr(kv), _dt(kv), kv.stride(0), _ptr(q), q.stride(0), _ptr(q_full), q_full.stride(0), _ptr(q_exp),
             q_exp.stride(0) if q_exp is not None else 0, _ptr(norm_w),
             float(eps), _ptr(inv_freq), int(rot_dims), _ptr(positions), _ptr(row_seq), _ptr(block_table),
             block_table.shape[1] if block_table is not None else 0, _ptr(k_cache), num_pages, page_size, T, num_seqs,
             H, dq, dr, rk, 1 if interleaved else 0, float(rot_scale), _ptr(status), _stream()),
           f"latent_prepare(rank={rk}, rot={dr})")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def activation(x, out, kind: str) -> None:
    """out = act(x) elementwise on rows (fp32 arithmetic); kinds: relu2 (the square of relu), gelu_tanh, silu, relu."""
    _cuda(x, out)
    _need(kind in ACTIVATIONS, f"activation: kind {kind!r} is not one of {sorted(ACTIVATIONS)}")
    _need(x.dim() == 2 and out.shape == x.shape and x.dtype == out.dtype and x.stride(1) == 1 and out.stride(1) == 1,
          "activation: x and out must be rows of the same shape and dtype")
    f = _fn("activation", "si_activation", [_c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(x), x.stride(0), _ptr(out), out.stride(0), _dt(x), x.shape[0], x.shape[1], ACTIVATIONS[kind], _stream()),
           f"activation({kind})")


# ---- state-space mixer ---------------------------------------------------------------------------------

def causal_conv(u, weight, bias, state, conv_off: int, out, positions, row_seq, q_start, ctx_len, slots,
                num_seqs: int, status=None) -> None:
    """out[t, c] (fp32) = silu(bias[c] + sum_k weight[c, k] * u[t - (K-1) + k, c]) per sequence, zeros before its
    start; inputs of earlier steps come from ``state[slot, conv_off:]`` ([K-1, C], fp32), which is renewed with
    this step's last K - 1 inputs afterwards (two launches)."""
    _cuda(u, weight, bias, state, out, positions, row_seq, q_start, ctx_len, slots, status)
    for t, nm in ((positions, "positions"), (row_seq, "row_seq"), (q_start, "q_start"), (ctx_len, "ctx_len"), (slots, "slots")):
        _i32(t, nm)
    T, C = u.shape
    K = weight.shape[1]
    _need(u.stride(1) == 1 and weight.shape == (C, K), "causal_conv: u must be rows [T, C], weight [C, K]")
    _f32v(weight, "weight"); _f32v(bias, "bias", C)
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, C), "causal_conv: out must be fp32 [T, C]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
          and state.shape[1] >= conv_off + (K - 1) * C, "causal_conv: state must be fp32 [slots, >= conv_off + (K-1)*C]")
    f = _fn("ssm", "si_causal_conv",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(u), _dt(u), u.stride(0), _ptr(weight), _ptr(bias), _ptr(state), state.stride(0), int(conv_off), _ptr(out),
             _ptr(positions), _ptr(row_seq), _ptr(q_start), _ptr(ctx_len), _ptr(slots), T, int(num_seqs), C, K,
             _ptr(status), _stream()), f"causal_conv(channels={C}, taps={K})", kernels=2 if K > 1 else 1)


def ssm_padded_state(N: int, P: int) -> int:
    """State rows per head as the scan kernel keeps them: N rounded up to (lanes per column) x (entries per lane). The
    same rule as ``scan_shape`` in ssm.cu, restated here so that a model's state size is known without the library;
    ``ssm_padded_state_of_library`` asks the library, and a test holds the two together."""
    ns = 32
    while ns > 1 and (P * ns > 1024 or ns * 2 > N):
        ns //= 2
    while ns > 1 and P * ns > 512 and -(-N // (ns // 2)) <= 16:
        ns //= 2
    while ns > 1 and -(-N // ns) < 4:
        ns //= 2
    per = -(-N // ns)
    if per > 32:
        raise KernelError(f"ssm_scan: a state of {N} x {P} is outside what the kernel supports")
    return ns * (4 if per <= 4 else 8 if per <= 8 else 16 if per <= 16 else 32)


def ssm_padded_state_of_library(N: int, P: int) -> int:
    lib = build.load("ssm")
    lib.si_ssm_padded_state.restype = _c_int
    return lib.si_ssm_padded_state(_c_int(N), _c_int(P))


def ssm_scan(xbc, dt_raw, dt_bias, a_log, d_skip, state, y, q_start, ctx_len, slots, num_seqs: int, heads: int,
             groups: int, N: int, P: int) -> None:
    """The recurrence over every sequence's rows of this step, from and into the first
    ``heads * ssm_padded_state(N, P) * P`` floats of ``state[slot]`` (fp32, in the kernel's own order; from zero for a
    portion that starts at position 0). ``xbc`` fp32 [T, heads*P + 2*groups*N] = [x | B | C];
    ``dt_raw`` [T, heads] (compute dtype, a strided view); ``y`` fp32 [T, heads*P]."""
    _cuda(xbc, dt_raw, dt_bias, a_log, d_skip, state, y, q_start, ctx_len, slots)
    for t, nm in ((q_start, "q_start"), (ctx_len, "ctx_len"), (slots, "slots")):
        _i32(t, nm)
    T = xbc.shape[0]
    _need(xbc.dtype == torch.float32 and xbc.stride(1) == 1 and xbc.shape[1] == heads * P + 2 * groups * N,
          "ssm_scan: xbc must be fp32 [T, heads*P + 2*groups*N]")
    _need(dt_raw.shape == (T, heads) and dt_raw.stride(1) == 1, "ssm_scan: dt_raw must be [T, heads]")
    _need(y.dtype == torch.float32 and y.shape == (T, heads * P) and y.stride(1) == 1, "ssm_scan: y must be fp32 [T, heads*P]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
          and state.shape[1] >= heads * ssm_padded_state(N, P) * P,
          "ssm_scan: state must be fp32 [slots, >= heads * ssm_padded_state(N, P) * P]")
    _f32v(dt_bias, "dt_bias", heads); _f32v(a_log, "a_log", heads); _f32v(d_skip, "d_skip", heads)
    f = _fn("ssm", "si_ssm_scan",
            [_c_p, _c_ll, _c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(xbc), xbc.stride(0), _ptr(dt_raw), _dt(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(a_log),
             _ptr(d_skip), _ptr(state), state.stride(0), _ptr(y), y.stride(0), _ptr(q_start), _ptr(ctx_len), _ptr(slots),
             int(num_seqs), heads, groups, N, P, _stream()), f"ssm_scan(heads={heads}, state={N}, head_dim={P})")


def gated_part_norm(y, z, weight, out, parts: int, eps: float) -> None:
    """out = g / sqrt(mean(g^2) + eps) * weight with g = y * silu(z), the mean over each of ``parts`` equal parts of a
    row. ``y`` fp32 rows, ``z`` and ``out`` rows in the compute dtype (views with a row stride are fine)."""
    _cuda(y, z, weight, out)
    T, W = y.shape
    _need(y.dtype == torch.float32 and y.stride(1) == 1 and z.shape == (T, W) and out.shape == (T, W)
          and z.stride(1) == 1 and out.stride(1) == 1 and z.dtype == out.dtype, "gated_part_norm: shapes or dtypes")
    _f32v(weight, "weight", W)
    f = _fn("ssm", "si_gated_part_norm", [_c_p, _c_ll, _c_p, _c_int, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_ptr(y), y.stride(0), _ptr(z), _dt(z), z.stride(0), _ptr(weight), _ptr(out), out.stride(0), T, W, int(parts),
             float(eps), _stream()), f"gated_part_norm(width={W}, parts={parts})")


# ---- general attention on the tensor cores (bf16) ---------------------------------------------------------

def attn_flex_ok(H: int, KV: int, dk: int, dv: int, own_v: bool) -> bool:
    lib = build.load("attention_flex")
    lib.si_attn_flex_ok.restype = _c_int
    return bool(lib.si_attn_flex_ok(_c_int(H), _c_int(KV), _c_int(dk), _c_int(dv), _c_int(1 if own_v else 0)))


def attn_flex_tokens(H: int, KV: int) -> int:
    """Most tokens of one work item of ``attn_flex``."""
    lib = build.load("attention_flex")
    lib.si_attn_flex_tokens.restype = _c_int
    return lib.si_attn_flex_tokens(_c_int(H), _c_int(KV))


def attn_flex_scratch_floats(num_items: int, H: int, KV: int, dv: int, nsplit: int) -> int:
    lib = build.load("attention_flex")
    lib.si_attn_flex_scratch_floats.restype = _c_llr
    return lib.si_attn_flex_scratch_floats(_c_int(num_items), _c_int(H), _c_int(KV), _c_int(dv), _c_int(nsplit))


def attn_flex(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int, KV: int, dk: int,
              dv: int, scale: float, window: int = 0, dist_bias=None, sink=None, nsplit: int = 1, scratch=None,
              status=None, max_rows: int = 0, softcap: float = 0.0, v_share: int = 1, slopes=None, q_temp=None, gate=None) -> None:
    """``attention_general`` on the tensor cores for bfloat16. ``items``: int32 [n, 4] rows (sequence, first row,
    tokens, first position) of at most ``attn_flex_tokens`` tokens. ``nsplit`` > 1 cuts every item's keys into that
    many shares (decode rows over long contexts); ``scratch`` then holds ``attn_flex_scratch_floats`` floats.
    ``max_rows``: the most rows (tokens x query heads of a key head served together) of any item when the caller knows it
    (0: unknown); at most 16 rows over keys that are their own values let a block's warps take a value slice each.
    ``softcap``, ``v_share``, ``slopes``, ``q_temp``, ``gate`` as in ``attention_general``; ``out`` may be fp32."""
    _cuda(q, k_cache, v_cache, block_table, items, out, dist_bias, sink, scratch, slopes, gate, status)
    _need(gate is None or (gate.dtype == torch.bfloat16 and gate.shape == (q.shape[0], H * dv) and gate.stride(1) == 1
                           and gate.stride(0) % 2 == 0 and gate.data_ptr() % 4 == 0), "attn_flex: gate must be bf16 [T, H*dv], rows 4-byte aligned")
    _f32v(slopes, "slopes", H)
    qt_coef, qt_every = _q_temp(q_temp)
    _i32(block_table, "block_table"); _i32(items, "items")
    _need(v_share >= 1 and KV % v_share == 0 and (v_share == 1 or v_cache is not None), "attn_flex: v_share")
    _need(q.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32) and k_cache.dtype == torch.bfloat16
          and (v_cache is None or v_cache.dtype == torch.bfloat16), "attn_flex: bfloat16 tensors only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * dk and out.shape[1] == H * dv,
          "attn_flex: q must be [T, H*dk], out [T, H*dv]")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, dk) and k_cache.is_contiguous(), "attn_flex: keys must be [pages, KV, page_size, dk]")
    if v_cache is not None:
        _need(tuple(v_cache.shape) == (k_cache.shape[0], KV // v_share, page_size, dv) and v_cache.is_contiguous(),
              "attn_flex: values must be [pages, KV / v_share, page_size, dv]")
    _need(items.dim() == 2 and items.shape[1] == 4, "attn_flex: items must be int32 [n, 4]")
    _need(q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and k_cache.data_ptr() % 16 == 0
          and (v_cache is None or v_cache.data_ptr() % 16 == 0) and out.data_ptr() % 8 == 0 and out.stride(0) % 2 == 0,
          "attn_flex: q and the caches must be 16-byte aligned")
    nd = 0
    if dist_bias is not None:
        _need(dist_bias.dim() == 2 and dist_bias.shape[1] == H, "attn_flex: dist_bias must be [nd, H]")
        _f32v(dist_bias, "dist_bias")
        nd = dist_bias.shape[0]
    _f32v(sink, "sink", H)
    if nsplit > 1:
        need = attn_flex_scratch_floats(items.shape[0], H, KV, dv, nsplit)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_flex: scratch must hold {need} floats")
    f = _fn("attention_flex", "si_attn_flex",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_f, _c_int, _c_int, _c_p, _c_f, _c_int,
             _c_p, _c_ll, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(items),
             items.shape[0], _ptr(out), out.stride(0), k_cache.shape[0], page_size, num_seqs, H, KV, dk, dv,
             float(scale), int(window or 0), _ptr(dist_bias), nd, _ptr(sink), int(nsplit), _ptr(scratch), int(max_rows),
             float(softcap or 0.0), int(v_share), 1 if out.dtype == torch.float32 else 0, _ptr(slopes), qt_coef, qt_every,
             _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(status), _stream()), f"attn_flex(heads={H}, kv_heads={KV}, dk={dk}, dv={dv})", kernels=2 if nsplit > 1 else 1)


# ---- one small matrix per head (decode rows) -----------------------------------------------------------------

def gemm_heads_ok(a, w, out, H: int, a_head: int, o_head: int) -> bool:
    """True when ``gemm_heads`` takes these tensors: bf16, at most 16 rows, K a multiple of 8, 16-byte aligned heads."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and a.shape[0] <= 16
            and w.dim() == 3 and w.shape[0] == H and w.is_contiguous() and w.shape[2] % 8 == 0 and a.stride(1) == 1
            and out.stride(1) == 1 and a.stride(0) % 8 == 0 and a_head % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and a.shape[0] * w.shape[2] * 2 <= 48 * 1024)


def gemm_heads(a, w, out, a_head: int, o_head: int) -> None:
    """out[t, h*o_head : h*o_head + N] = a[t, h*a_head : h*a_head + K] @ w[h]^T for every head h of w [H, N, K], at
    most 16 rows, in one launch (``a_head``, ``o_head``: distance between heads within a row, in elements)."""
    _cuda(a, w, out)
    H, N, K = w.shape
    M = a.shape[0]
    _need(gemm_heads_ok(a, w, out, H, a_head, o_head), "gemm_heads: bf16, at most 16 rows, K a multiple of 8, aligned heads")
    _need(out.shape[0] == M and a.shape[1] >= (H - 1) * a_head + K and out.shape[1] >= (H - 1) * o_head + N, "gemm_heads: shapes")
    f = _fn("gemm_heads", "si_gemm_heads", [_c_p, _c_ll, _c_ll, _c_p, _c_p, _c_ll, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), int(a_head), _ptr(w), _ptr(out), out.stride(0), int(o_head), M, H, N, K, _stream()),
           f"gemm_heads(M={M}, heads={H}, N={N}, K={K})")


def latent_gather(k_cache, block_table, seqs, max_keys: int, dense, page_size: int, num_seqs: int, status=None) -> None:
    """Copies the cached rows of positions first .. first + keys - 1 of the listed sequences out of the pages into consecutive
    rows of ``dense`` [rows, width]. ``seqs``: int32 [E, 4] rows of (sequence of the step, first dense row, keys, first position);
    ``max_keys``: the most keys of any of them. ``k_cache`` [pages, 1, page_size, width]."""
    _cuda(k_cache, block_table, seqs, dense, status)
    _i32(block_table, "block_table"); _i32(seqs, "seqs")
    width = k_cache.shape[3]
    _need(k_cache.is_contiguous() and k_cache.shape[1] == 1 and k_cache.shape[2] == page_size and dense.is_contiguous()
          and dense.shape[1] == width and dense.dtype == k_cache.dtype and seqs.dim() == 2 and seqs.shape[1] == 4,
          "latent_gather: cache [pages, 1, page_size, width], dense [rows, width], seqs [E, 4]")
    f = _fn("attention_general", "si_latent_gather",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(k_cache), _dt(k_cache), _ptr(block_table), block_table.shape[1], _ptr(seqs), seqs.shape[0], int(max_keys),
             _ptr(dense), k_cache.shape[0], page_size, int(num_seqs), width, _ptr(status), _stream()), "latent_gather")


def latent_expand_keys(plain, dense, keys, H: int, dq: int, dr: int, rk: int) -> None:
    """keys[t, h] = [plain[t, h*dq:(h+1)*dq] | dense[t, rk:rk+dr]] for every row t: per-head keys from the expanded plain
    parts [rows, H*dq] and the shared rotated part that the gathered rows [rows, rk+dr] end with."""
    _cuda(plain, dense, keys)
    rows = plain.shape[0]
    _need(plain.is_contiguous() and dense.is_contiguous() and keys.is_contiguous() and plain.shape == (rows, H * dq)
          and dense.shape == (rows, rk + dr) and keys.numel() == rows * H * (dq + dr) and plain.dtype == dense.dtype == keys.dtype,
          "latent_expand_keys: shapes or dtypes")
    f = _fn("attention_general", "si_latent_expand_keys", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(plain), _ptr(dense), _ptr(keys), _dt(plain), rows, H, dq, dr, rk, _stream()), "latent_expand_keys")


# ---- queries and keys with a norm and a rotation of their own; differential attention -----------------------------

def qk_prepare(rows, q_weight, k_weight, eps: float, inv_freq, rot_dims: int, interleaved: bool, positions, row_seq,
               block_table, k_cache, v_cache, page_size: int, num_seqs: int, NQ: int, NK: int, NV: int, dk: int, dv: int,
               status=None, q_out=None, maps: int = 1, whole: bool = False, rot_scale: float = 1.0) -> None:
    """Rows ``[q: NQ*dk | k: NK*dk | v: NV*dv | ...]`` of a stacked projection: every q and k vector is RMS-normalised
    (shared fp32 weights ``q_weight``, ``k_weight`` [dk]; None: no norm), its first ``rot_dims`` entries rotated by the
    row's position (pairs (2i, 2i+1) if ``interleaved``, else (i, i + rot_dims/2); angle pos * inv_freq[i]); q in place
    or into ``q_out`` [T, NQ*dk], k into ``k_cache`` [pages, NK, page_size, dk], v into ``v_cache`` [pages, NV, page_size, dv]
    (None: nothing stored). ``maps`` M > 1: the q and k vectors of a head come as M maps, [head][map], and ``q_out`` (needed
    then) is ordered [key head][map][head of the group], so that query vector i reads key vector i // (NQ / NK)."""
    _cuda(rows, q_weight, k_weight, inv_freq, positions, row_seq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    _need(rows.dim() == 2 and rows.stride(1) == 1 and rows.shape[1] >= (NQ + NK) * dk + NV * dv, "qk_prepare: row layout")
    _f32v(q_weight, "q_weight", NQ * dk if whole else dk); _f32v(k_weight, "k_weight", NK * dk if whole else dk)
    _need(not whole or maps == 1, "qk_prepare: a norm over the whole projection goes without maps")
    _f32v(inv_freq, "inv_freq")
    _need(rot_dims == 0 or (inv_freq is not None and inv_freq.numel() >= rot_dims // 2), "qk_prepare: inv_freq too short")
    if q_out is None:
        _need(maps == 1, "qk_prepare: maps need q_out")
        q_out = rows
    else:
        _cuda(q_out)
        _need(q_out.dtype == rows.dtype and q_out.dim() == 2 and q_out.stride(1) == 1 and q_out.shape == (rows.shape[0], NQ * dk),
              "qk_prepare: q_out must be [T, NQ*dk]")
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == rows.dtype and k_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (NK, page_size, dk)
              and v_cache is not None and v_cache.dtype == rows.dtype and v_cache.is_contiguous()
              and tuple(v_cache.shape) == (k_cache.shape[0], NV, page_size, dv),
              "qk_prepare: caches must be [pages, NK, page_size, dk] and [pages, NV, page_size, dv]")
        num_pages = k_cache.shape[0]
    f = _fn("qk_prepare", "si_qk_prepare",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_f, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_f, _c_p, _c_p])
    _check(f(_ptr(rows), _dt(rows), rows.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq), int(rot_dims),
             1 if interleaved else 0, _ptr(positions), _ptr(row_seq), _ptr(block_table),
             block_table.shape[1] if block_table is not None else 0, _ptr(k_cache), _ptr(v_cache), num_pages, page_size,
             rows.shape[0], int(num_seqs), NQ, NK, NV, dk, dv, _ptr(q_out), q_out.stride(0), int(maps), 1 if whole else 0,
             float(rot_scale), _ptr(status), _stream()),
           f"qk_prepare(dk={dk}, dv={dv})")


def diff_combine(a, gate, out, H: int, dv: int, ratio: int, lam: float, eps: float, post: float) -> None:
    """``a`` [T, H*2*dv] (fp32 or the compute dtype) holds the two maps' results in the order [key head][map][head of the
    group] (``ratio`` heads a key head): per head o = a0 - lam * a1, divided by its root mean square (eps inside the
    root), times ``post``, times sigmoid(gate[t, h]) (``gate`` [T, H], a strided view; None: no gate); ``out`` [T, H*dv]."""
    _cuda(a, gate, out)
    T = a.shape[0]
    _need(a.shape == (T, H * 2 * dv) and a.stride(1) == 1 and out.shape == (T, H * dv) and out.stride(1) == 1, "diff_combine: shapes")
    _need(a.dtype in (out.dtype, torch.float32), "diff_combine: dtypes")
    if gate is not None:
        _need(gate.shape == (T, H) and gate.stride(1) == 1 and gate.dtype == out.dtype, "diff_combine: gate must be [T, H]")
    f = _fn("qk_prepare", "si_diff_combine",
            [_c_p, _c_int, _c_ll, _c_p, _c_ll, _c_p, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_f, _c_f, _c_f, _c_p])
    _check(f(_ptr(a), _dt(a), a.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), _dt(out),
             out.stride(0), T, H, dv, int(ratio), float(lam), float(eps), float(post), _stream()), f"diff_combine(heads={H}, dv={dv})")


def talk_combine(a, talk, gate, out, H: int, G: int, dv: int, post: float = 1.0) -> None:
    """Attention weights mixed over the heads, applied after the fact: ``a`` [T, H*G*dv] (fp32 or the compute dtype) holds
    for every query head what its weights give on the values of each of the G key/value heads; out[t, h, :] =
    post * sigmoid(gate[t, h, :]) * sum_g talk[h, g] * a[t, g, kv(h), :] with kv(h) = h // (H / G). ``talk`` fp32 [H, H],
    ``gate`` [T, H*dv] in ``out``'s dtype (a strided view; None: no gate), ``out`` [T, H*dv] (a strided view)."""
    _cuda(a, talk, gate, out)
    T = a.shape[0]
    _need(a.shape == (T, H * G * dv) and a.stride(1) == 1 and out.shape == (T, H * dv) and out.stride(1) == 1, "talk_combine: shapes")
    _need(a.dtype in (out.dtype, torch.float32), "talk_combine: dtypes")
    _f32v(talk, "talk", H * H)
    if gate is not None:
        _need(gate.shape == (T, H * dv) and gate.stride(1) == 1 and gate.dtype == out.dtype, "talk_combine: gate must be [T, H*dv]")
    f = _fn("qk_prepare", "si_talk_combine",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_ll, _c_p, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_ptr(a), _dt(a), a.stride(0), _ptr(talk), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
             _dt(out), out.stride(0), T, H, G, dv, float(post), _stream()), f"talk_combine(heads={H}, dv={dv})")


# ---- time mixing with a decaying matrix state ------------------------------------------------------------------------

def shift_mix(x, mu, out, state, prev_off: int, positions, row_seq, q_start, slots, num_seqs: int, status=None) -> None:
    """out[m, t, :] = x[t] + (x[t - 1] - x[t]) * mu[m] for every row t, where x[t - 1] is the row before in the same
    sequence: the step's own, or for a portion's first row ``state[slot, prev_off:prev_off + d]`` (zeros at position 0),
    which is then renewed with the portion's last row. ``x`` [T, d] (rows may have a stride), ``mu`` fp32 [M, d], ``out``
    contiguous [M, T, d] in x's dtype, ``state`` fp32 [slots, n]."""
    _cuda(x, mu, out, state, positions, row_seq, q_start, slots, status)
    for t, nm in ((positions, "positions"), (row_seq, "row_seq"), (q_start, "q_start"), (slots, "slots")):
        _i32(t, nm)
    T, d = x.shape
    M = mu.shape[0]
    _need(x.stride(1) == 1 and out.shape == (M, T, d) and out.is_contiguous() and out.dtype == x.dtype, "shift_mix: out must be [M, T, d]")
    _f32v(mu, "mu", M * d)
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and prev_off + d <= state.shape[1],
          "shift_mix: state must be fp32 [slots, >= prev_off + d]")
    f = _fn("time_mix", "si_shift_mix", [_c_p, _c_int, _c_ll, _c_p, _c_int, _c_p, _c_ll, _c_p, _c_ll, _c_ll, _c_p, _c_p, _c_p, _c_p,
                                         _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(x), _dt(x), x.stride(0), _ptr(mu), M, _ptr(out), T * d, _ptr(state), state.stride(0), int(prev_off),
             _ptr(positions), _ptr(row_seq), _ptr(q_start), _ptr(slots), T, int(num_seqs), d, _ptr(status), _stream()),
           f"shift_mix(d={d})")


def time_mix_prepare(r, k, v, z, w2t, w0, xs) -> None:
    """``xs`` fp32 [T, 4C] = [r | k | v | decay] with decay = exp(-exp(tanh(z) @ w2t + w0)): ``r``, ``k``, ``v`` [T, C] and
    ``z`` [T, L] in the compute dtype (views with a row stride), ``w2t`` fp32 [L, C], ``w0`` fp32 [C]."""
    _cuda(r, k, v, z, w2t, w0, xs)
    T, C = r.shape
    L = z.shape[1]
    _need(k.shape == (T, C) and v.shape == (T, C) and z.shape[0] == T and all(t.stride(1) == 1 for t in (r, k, v, z))
          and r.dtype == k.dtype == v.dtype == z.dtype, "time_mix_prepare: r, k, v must be [T, C] and z [T, L] of one dtype")
    _f32v(w2t, "w2t", L * C); _f32v(w0, "w0", C)
    _need(xs.dtype == torch.float32 and xs.is_contiguous() and xs.shape == (T, 4 * C), "time_mix_prepare: xs must be fp32 [T, 4C]")
    f = _fn("time_mix", "si_time_mix_prepare", [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_p, _c_p, _c_p,
                                                _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(r), r.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(z), z.stride(0), _dt(r), _ptr(w2t), _ptr(w0),
             _ptr(xs), T, C, L, _stream()), f"time_mix_prepare(C={C}, L={L})")


def decay_state_floats(n: int) -> int:
    """fp32 entries of one head's n x n state as ``decay_scan`` keeps it in a slot ([rows a thread][n][parts a column], the
    rows padded to rows a thread x parts): the rule of ``decay_shape`` in time_mix.cu, restated so that a model's state size
    is known without the library; ``decay_state_floats_of_library`` asks the library, and a test holds the two together."""
    if n <= 0 or n > 512:
        raise KernelError(f"decay_scan: a state of {n} x {n} is outside what the kernel supports")
    r = (-(-n // 16) + 3) // 4 * 4
    parts = 1
    while parts * r < n:
        parts *= 2
    return r * parts * n


def decay_state_floats_of_library(n: int) -> int:
    lib = build.load("time_mix")
    lib.si_decay_state_floats.restype = _c_ll
    return lib.si_decay_state_floats(_c_int(n))


def decay_scan(xs, u, state, y, q_start, ctx_len, slots, num_seqs: int, H: int, n: int) -> None:
    """Per head o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(decay_t) S + k_t v_t^T, over every sequence's rows of
    this step, from and into the first ``H * decay_state_floats(n)`` floats of ``state[slot]`` (fp32, in the kernel's own
    order; from zero for a portion that starts at position 0). ``xs`` fp32 [T, 4*H*n] = [r | k | v | decay] as
    ``time_mix_prepare`` leaves it, ``u`` fp32 [H, n], ``y`` fp32 [T, H*n]."""
    _cuda(xs, u, state, y, q_start, ctx_len, slots)
    for t, nm in ((q_start, "q_start"), (ctx_len, "ctx_len"), (slots, "slots")):
        _i32(t, nm)
    T = xs.shape[0]
    _need(xs.dtype == torch.float32 and xs.stride(1) == 1 and xs.shape[1] == 4 * H * n, "decay_scan: xs must be fp32 [T, 4*H*n]")
    _need(y.dtype == torch.float32 and y.shape == (T, H * n) and y.stride(1) == 1, "decay_scan: y must be fp32 [T, H*n]")
    _f32v(u, "u", H * n)
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
          and state.shape[1] >= H * decay_state_floats(n), "decay_scan: state must be fp32 [slots, >= H * decay_state_floats(n)]")
    f = _fn("time_mix", "si_decay_scan", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(xs), xs.stride(0), _ptr(u), _ptr(state), state.stride(0), _ptr(y), y.stride(0), _ptr(q_start), _ptr(ctx_len),
             _ptr(slots), int(num_seqs), H, n, _stream()), f"decay_scan(heads={H}, n={n})")


# ---- gated delta rule ------------------------------------------------------------------------------------------------

def delta_state_floats(dk: int, dv: int) -> int:
    """fp32 entries of one head's dk x dv state as the scan kernel keeps it in a slot ([rows a thread][dv][parts a column],
    the rows padded to rows a thread x parts). The same rule as ``delta_shape`` in delta_rule.cu, restated here so that a
    model's state size is known without the library; ``delta_state_floats_of_library`` asks the library, and a test holds
    the two together."""
    if dk <= 0 or dv <= 0 or dk > 512:
        raise KernelError(f"delta_scan: a state of {dk} x {dv} is outside what the kernel supports")
    r = (-(-dk // 16) + 3) // 4 * 4
    parts = 1
    while parts * r < dk:
        parts *= 2
    return r * parts * dv


def delta_state_floats_of_library(dk: int, dv: int) -> int:
    lib = build.load("delta_rule")
    lib.si_delta_state_floats.restype = _c_ll
    return lib.si_delta_state_floats(_c_int(dk), _c_int(dv))


def delta_prepare(xc, ba, b_off: int, a_off: int, a_log, dt_bias, bg, G: int, H: int, dk: int, q_scale: float) -> None:
    """``xc`` fp32 rows [q: G*dk | k: G*dk | ...]: q and k become unit vectors per head (x / sqrt(sum(x^2) + 1e-6)), q times
    ``q_scale``. ``ba``: rows holding H raw values b at column ``b_off`` and H raw values a at ``a_off``;
    ``bg`` fp32 [T, 2H + G] receives beta = sigmoid(b), g = exp(-exp(a_log) * softplus(a + dt_bias)) and, per query/key
    head, q . k of the prepared vectors."""
    _cuda(xc, ba, a_log, dt_bias, bg)
    T = xc.shape[0]
    _need(xc.dtype == torch.float32 and xc.stride(1) == 1 and xc.shape[1] >= 2 * G * dk, "delta_prepare: xc must be fp32 rows")
    _need(ba.shape[0] == T and ba.stride(1) == 1 and ba.shape[1] >= max(b_off, a_off) + H, "delta_prepare: ba rows")
    _need(bg.dtype == torch.float32 and bg.is_contiguous() and bg.shape == (T, 2 * H + G), "delta_prepare: bg must be fp32 [T, 2H + G]")
    _f32v(a_log, "a_log", H); _f32v(dt_bias, "dt_bias", H)
    f = _fn("delta_rule", "si_delta_prepare",
            [_c_p, _c_ll, _c_p, _c_int, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(f(_ptr(xc), xc.stride(0), _ptr(ba), _dt(ba), ba.stride(0), int(b_off), int(a_off), _ptr(a_log), _ptr(dt_bias),
             _ptr(bg), T, G, H, dk, float(q_scale), _stream()), f"delta_prepare(heads={H})")


def delta_scan(xc, bg, state, y, q_start, ctx_len, slots, num_seqs: int, G: int, H: int, dk: int, dv: int) -> None:
    """The gated delta rule over every sequence's rows of this step: per head S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q, from and into the first ``H * delta_state_floats(dk, dv)`` floats of ``state[slot]`` (fp32,
    in the kernel's own order; from zero for a portion that starts at position 0). ``xc`` fp32 [T, 2*G*dk + H*dv] =
    [q | k | v] and ``bg`` fp32 [T, 2H + G] as ``delta_prepare`` leaves them, ``y`` fp32 [T, H*dv]. Head h reads q/k
    head h // (H / G)."""
    _cuda(xc, bg, state, y, q_start, ctx_len, slots)
    for t, nm in ((q_start, "q_start"), (ctx_len, "ctx_len"), (slots, "slots")):
        _i32(t, nm)
    T = xc.shape[0]
    _need(xc.dtype == torch.float32 and xc.stride(1) == 1 and xc.shape[1] >= 2 * G * dk + H * dv, "delta_scan: xc must be fp32 [T, 2*G*dk + H*dv]")
    _need(bg.dtype == torch.float32 and bg.is_contiguous() and bg.shape == (T, 2 * H + G), "delta_scan: bg must be fp32 [T, 2H + G]")
    _need(y.dtype == torch.float32 and y.shape == (T, H * dv) and y.stride(1) == 1, "delta_scan: y must be fp32 [T, H*dv]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
          and state.shape[1] >= H * delta_state_floats(dk, dv),
          "delta_scan: state must be fp32 [slots, >= H * delta_state_floats(dk, dv)]")
    f = _fn("delta_rule", "si_delta_scan",
            [_c_p, _c_ll, _c_p, _c_int, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(xc), xc.stride(0), _ptr(bg), bg.shape[1], _ptr(state), state.stride(0), _ptr(y), y.stride(0), _ptr(q_start),
             _ptr(ctx_len), _ptr(slots), int(num_seqs), G, H, dk, dv, _stream()), f"delta_scan(heads={H}, dk={dk}, dv={dv})")


def head_norm_gate(o, z, weight, out, H: int, dv: int, eps: float, post: float = 1.0) -> None:
    """out[t, h, :] = post * weight * o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * silu(z[t, h, :]); ``o`` fp32 [T, H*dv],
    ``z`` and ``out`` [T, H*dv] in the compute dtype (views with a row stride are fine), ``weight`` fp32 [dv] (shared by
    the heads) or [H*dv] (a row a head)."""
    _cuda(o, z, weight, out)
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.shape == (T, H * dv) and o.stride(1) == 1 and z.shape == (T, H * dv)
          and out.shape == (T, H * dv) and z.stride(1) == 1 and out.stride(1) == 1 and z.dtype == out.dtype,
          "head_norm_gate: shapes or dtypes")
    per_head = weight.numel() == H * dv and H > 1
    _f32v(weight, "weight", H * dv if per_head else dv)
    f = _fn("delta_rule", "si_head_norm_gate", [_c_p, _c_ll, _c_p, _c_int, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_f,
                                                 _c_ll, _c_f, _c_p])
    _check(f(_ptr(o), o.stride(0), _ptr(z), _dt(z), z.stride(0), _ptr(weight), _ptr(out), out.stride(0), T, H, dv, float(eps),
             dv if per_head else 0, float(post), _stream()), f"head_norm_gate(heads={H}, dv={dv})")


# ---- small elementwise steps -----------------------------------------------------------------------------------------

def softcap(x, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (contiguous fp32)."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "softcap: contiguous fp32 only")
    f = _fn("activation", "si_softcap", [_c_p, _c_ll, _c_f, _c_p])
    _check(f(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


def add_bias(x, bias) -> None:
    """x[t, :] += bias (fp32 [width]) in place; rows may have a stride."""
    _cuda(x, bias)
    _need(x.dim() == 2 and x.stride(1) == 1, "add_bias: x must be rows")
    _f32v(bias, "bias", x.shape[1])
    f = _fn("activation", "si_add_bias", [_c_p, _c_ll, _c_int, _c_p, _c_int, _c_int, _c_p])
    _check(f(_ptr(x), x.stride(0), _dt(x), _ptr(bias), x.shape[0], x.shape[1], _stream()), "add_bias")


def glu_limited(gu, bias, out, group, limit: float, alpha: float) -> None:
    """out[t, f] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate + bias, limit), u = clamp(up + bias, -limit, limit);
    ``gu`` [T, 2F] holds gate and up interleaved in groups of ``group`` columns (None: F), ``bias`` fp32 [2F] in the same
    order or None."""
    _cuda(gu, bias, out)
    T, F = out.shape
    _need(gu.shape == (T, 2 * F) and gu.is_contiguous() and out.is_contiguous() and gu.dtype == out.dtype, "glu_limited: gu must be [T, 2F]")
    _f32v(bias, "bias", 2 * F)
    f = _fn("swiglu", "si_glu_limited", [_c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_f, _c_p])
    _check(f(_ptr(gu), _ptr(bias), _ptr(out), _dt(out), T, F, F if group is None else int(group), float(limit), float(alpha),
             _stream()), f"glu_limited(F={F})")


# ---- routed feed-forward (mixture of experts) ----------------------------------------------------------------------------

MOE_ACTS = {"none": 0, "relu2": 1, "silu": 2, "gelu_tanh": 3, "glu_limited": 4}
MOE_SCORES = {"sigmoid": 0, "softmax": 1}


def moe_route(x, w, E: int, top: int, scale: float, ids, wts, gates=None, scores: str = "sigmoid", renorm: bool = False,
              choice_bias=None) -> None:
    """Scores of ``E`` experts for every row and the ``top`` largest: ``w`` [E + extra, d] holds the router's rows and
    behind them ``extra`` gate rows; ``ids`` int32 [T, top], ``wts`` fp32 [T, top] = score * scale (``renorm``: divided by
    the chosen scores' sum first), ``gates`` fp32 [T, extra] = sigmoid(w_gate . x). Scores are sigmoid(z) or softmax(z) of
    z = w x, summed in fp32 whatever the storage. ``choice_bias`` (fp32 [E]): the ``top`` largest of score + bias are chosen;
    the weights are still made of the scores alone."""
    _cuda(x, w, ids, wts, gates, choice_bias)
    _f32v(choice_bias, "choice_bias", E)
    T, d = x.shape
    extra = w.shape[0] - E
    _need(x.stride(1) == 1 and w.is_contiguous() and w.shape[1] == d and w.dtype == x.dtype and extra >= 0, "moe_route: x [T, d], w [E + extra, d]")
    _need(scores in MOE_SCORES, f"moe_route: scores {scores!r} is not one of {sorted(MOE_SCORES)}")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (T, top), "moe_route: ids must be int32 [T, top]")
    _need(wts.dtype == torch.float32 and wts.is_contiguous() and wts.shape == (T, top), "moe_route: wts must be fp32 [T, top]")
    if extra:
        _need(gates is not None and gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape == (T, extra),
              "moe_route: gates must be fp32 [T, extra]")
    f = _fn("moe", "si_moe_route", [_c_p, _c_int, _c_ll, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p,
                                    _c_p, _c_p, _c_int, _c_p])
    _check(f(_ptr(x), _dt(x), x.stride(0), _ptr(w), E, extra, d, top, float(scale), MOE_SCORES[scores], 1 if renorm else 0,
             _ptr(choice_bias), _ptr(ids), _ptr(wts), _ptr(gates), T, _stream()), f"moe_route(experts={E}, top={top})")


MOE_PLAN_CHUNK = 1024


def moe_plan_ints(P: int, E: int) -> int:
    """int32 entries of ``moe_plan``'s scratch for P pairs and E experts (ranks, then counts per chunk of 1,024 pairs)."""
    return P + -(-P // MOE_PLAN_CHUNK) * E


def moe_plan(ids, E: int, scratch, offsets, row_of, place_of) -> None:
    """The (row, choice) pairs of ``ids`` [T, top] ordered by expert, rows in their own order within an expert:
    ``offsets`` int32 [E + 1] (first place of every expert), ``row_of`` int32 [T*top] (the row at every place),
    ``place_of`` int32 [T, top] (the place of every pair); ``scratch`` int32 [moe_plan_ints(T*top, E)]."""
    _cuda(ids, scratch, offsets, row_of, place_of)
    T, top = ids.shape
    P = T * top
    for t, nm in ((ids, "ids"), (scratch, "scratch"), (offsets, "offsets"), (row_of, "row_of"), (place_of, "place_of")):
        _i32(t, nm)
    _need(scratch.numel() >= moe_plan_ints(P, E) and offsets.numel() == E + 1 and row_of.numel() == P and place_of.numel() == P,
          "moe_plan: sizes")
    f = _fn("moe", "si_moe_plan", [_c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p])
    _check(f(_ptr(ids), P, E, top, _ptr(scratch), _ptr(offsets), _ptr(row_of), _ptr(place_of), _stream()), f"moe_plan(experts={E})",
           kernels=1 if P <= MOE_PLAN_CHUNK else 3)


GROUPED_TC05_MIN_PLACES = 128      # fewer places than this (decode rows, short portions) stay on the mma.sync tiles
_GROUPED_TC05_ACTS = {"none": 0, "relu2": 1, "glu_limited": 2}


def moe_gemm_grouped_ok(a, w, out, P: int, act: str = "none") -> bool:
    """True when ``moe_gemm`` sends this product to the tcgen05 grouped kernel (bf16, many places, K a multiple of 8);
    a product that gathers its rows then wants the ``gathered`` scratch [P, K]."""
    E, N, K = w.shape
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and P >= max(GROUPED_TC05_MIN_PLACES, 8 * E)
            and act in _GROUPED_TC05_ACTS and (act == "none" or out.dtype == torch.bfloat16) and K % 8 == 0
            and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()
            and (P + 127) // 128 + E <= 1024 and gemm_tc05_available())


def moe_gather(a, rows, out) -> None:
    """out[p, :] = a[rows[p], :]: ``a`` [T, K] (rows may have a stride), ``rows`` int32 [P], ``out`` [P, K] of a's dtype."""
    _cuda(a, rows, out)
    _i32(rows, "rows")
    P, K = out.shape
    _need(a.dim() == 2 and a.shape[1] == K and a.stride(1) == 1 and out.stride(1) == 1 and out.dtype == a.dtype
          and rows.numel() == P, "moe_gather: a [T, K], rows [P], out [P, K]")
    f = _fn("moe", "si_moe_gather", [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), _dt(a), a.stride(0), _ptr(rows), _ptr(out), out.stride(0), P, a.shape[0], K, _stream()), f"moe_gather(K={K})")


def moe_gemm_tc05(a, w, out, offsets, act: str = "none", status=None, limit: float = 0.0, alpha: float = 1.702) -> None:
    """The grouped product on the tcgen05 tensor cores: out[p, :] = act(a[p, :] @ w[e]^T) for the places p of expert e
    (``a`` [P, K] already in the order of the places; ``moe_gemm_grouped_ok`` says when it may be called)."""
    _cuda(a, w, out, offsets, status)
    _i32(offsets, "offsets")
    E, N, K = w.shape
    P = out.shape[0]
    _need(a.shape == (P, K) and a.stride(1) == 1 and out.shape == (P, N // 2 if act == "glu_limited" else N) and out.stride(1) == 1
          and offsets.numel() >= E + 1, "moe_gemm_tc05: a [P, K], w [E, N, K], out [P, N] (glu_limited: [P, N / 2])")
    _need(moe_gemm_grouped_ok(a, w, out, P, act), "moe_gemm_tc05: bf16, at least 128 places, K a multiple of 8, aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_grouped", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int,
                                                  _c_int, _c_f, _c_f, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _weight_map(w.view(E * N, K)), _ptr(out), out.stride(0), _dt(out), _ptr(offsets), P, E, N, K,
             _GROUPED_TC05_ACTS[act], float(limit), float(alpha), _ptr(status), _stream()), f"moe_gemm_tc05(experts={E}, N={N}, K={K})")


def moe_gemm_tiles(a, a_rows, w, out, offsets, act: str = "none", limit: float = 0.0, alpha: float = 1.702) -> None:
    """``moe_gemm`` on the mma.sync tiles (bf16) or in true 32-bit, whatever the number of places."""
    _cuda(a, a_rows, w, out, offsets)
    _i32(a_rows, "a_rows"); _i32(offsets, "offsets")
    _need(act in MOE_ACTS, f"moe_gemm: act {act!r} is not one of {sorted(MOE_ACTS)}")
    E, N, K = w.shape
    P = out.shape[0]
    _need(a.dim() == 2 and a.shape[1] == K and a.stride(1) == 1 and w.is_contiguous() and w.dtype == a.dtype, "moe_gemm: a [*, K], w [E, N, K]")
    pair = act == "glu_limited"                       # gate and up rows in turn: an entry of the result for every two rows
    _need(not pair or (N % 2 == 0 and limit > 0), "moe_gemm: glu_limited needs an even N and a positive limit")
    _need(out.shape == (P, N // 2 if pair else N) and out.stride(1) == 1 and out.dtype in (a.dtype, torch.float32),
          "moe_gemm: out must be [P, N] (glu_limited: [P, N / 2])")
    _need(offsets.numel() >= E + 1 and (a_rows is None or a_rows.numel() == P) and (a_rows is not None or a.shape[0] >= P), "moe_gemm: sizes")
    f = _fn("moe", "si_moe_gemm", [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_ll, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                   _c_f, _c_f, _c_p])
    _check(f(_ptr(a), _dt(a), a.stride(0), _ptr(a_rows), _ptr(w), _ptr(out), _dt(out), out.stride(0), _ptr(offsets), P, E, N, K,
             MOE_ACTS[act], float(limit), float(alpha), _stream()), f"moe_gemm(experts={E}, N={N}, K={K})")


def moe_gemm(a, a_rows, w, out, offsets, act: str = "none", gathered=None, status=None, limit: float = 0.0,
             alpha: float = 1.702) -> None:
    """out[p, :] = act(a[row(p), :] @ w[e]^T) for every place p of expert e (``offsets`` int32 [E + 1] as ``moe_plan``
    leaves them); row(p) = a_rows[p] (int32 [P]) or p itself (None). ``a`` [*, K] and ``w`` [E, N, K] of one dtype;
    ``out`` [P, N] in that dtype or fp32. bf16 on the tensor cores with fp32 sums (tcgen05 where ``moe_gemm_grouped_ok``;
    a product that gathers then copies its rows into ``gathered`` [P, K] first), fp32 in true 32-bit. ``offsets`` may hold
    more entries than E + 1 (experts behind the E that have weights, which get no product); places behind offsets[E] are
    left alone. act "glu_limited": ``w`` holds gate and up rows in turn and ``out`` is [P, N / 2] (``limit``, ``alpha``)."""
    P = out.shape[0]
    if moe_gemm_grouped_ok(a, w, out, P, act) and (a_rows is None or gathered is not None):
        if a_rows is not None:
            moe_gather(a, a_rows, gathered)
            a = gathered
        moe_gemm_tc05(a[:P], w, out, offsets, act, status, limit, alpha)
    else:
        moe_gemm_tiles(a, a_rows, w, out, offsets, act, limit, alpha)


def moe_combine(y, place_of, wts, out, shared=None, gate=None, ids=None, real: int = 0, x=None) -> None:
    """out[t, :] = sum_c wts[t, c] * y[place_of[t, c], :] (+ gate[t] * shared[t, :]): ``y`` [P, d] (fp32 or out's dtype),
    ``place_of`` int32 [T, top], ``wts`` fp32 [T, top], ``shared`` [T, d] in out's dtype or None, ``gate`` fp32 [T] (a strided
    view; None: 1), ``out`` [T, d]. With ``ids`` (int32 [T, top]) a choice whose id is ``real`` or above is an identity expert:
    its result is the row ``x[t]`` itself (``x`` [T, d] in out's dtype) and ``y`` is not read there."""
    _cuda(y, place_of, wts, out, shared, gate, ids, x)
    if ids is not None:
        _i32(ids, "ids")
        _need(ids.shape == tuple(place_of.shape) and ids.is_contiguous() and x is not None and x.shape == tuple(out.shape)
              and x.stride(1) == 1 and x.dtype == out.dtype, "moe_combine: ids [T, top] with x [T, d]")
    _i32(place_of, "place_of")
    T, d = out.shape
    top = wts.shape[1]
    _need(y.shape[1] == d and y.stride(1) == 1 and out.stride(1) == 1 and y.dtype in (out.dtype, torch.float32), "moe_combine: y [P, d]")
    _need(place_of.shape == (T, top) and wts.shape == (T, top) and wts.dtype == torch.float32 and wts.is_contiguous(), "moe_combine: wts, place_of")
    if shared is not None:
        _need(shared.shape == (T, d) and shared.stride(1) == 1 and shared.dtype == out.dtype, "moe_combine: shared must be [T, d]")
    if gate is not None:
        _need(shared is not None and gate.dtype == torch.float32 and gate.dim() == 1 and gate.shape[0] == T, "moe_combine: gate must be fp32 [T]")
    f = _fn("moe", "si_moe_combine", [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_int, _c_p, _c_ll, _c_p, _c_int, _c_p, _c_int, _c_ll, _c_int, _c_int,
                                      _c_p, _c_int, _c_p, _c_ll, _c_p])
    _check(f(_ptr(y), _dt(y), y.stride(0), _ptr(place_of), _ptr(wts), top, _ptr(shared), shared.stride(0) if shared is not None else 0,
             _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), _dt(out), out.stride(0), T, d,
             _ptr(ids) if ids is not None else None, int(real), _ptr(x) if ids is not None else None,
             x.stride(0) if ids is not None else 0, _stream()),
           f"moe_combine(d={d})")


# ---- gated sublayers into the stream ---------------------------------------------------------------------------------------

def gated_add(resid, z1, b1, a, z2=None, b2=None, f=None, mult: float = 1.0) -> None:
    """resid (fp32, in place) += mult * (sigmoid(z1 + b1) * a + sigmoid(z2 + b2) * f); the second sublayer may be absent.
    ``z``, ``a``, ``f`` contiguous [T, d] of one dtype, ``b`` fp32 [d]."""
    _cuda(resid, z1, b1, a, z2, b2, f)
    T, d = resid.shape
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "gated_add: resid must be contiguous fp32 rows")
    for t in (z1, a, z2, f):
        _need(t is None or (t.shape == (T, d) and t.is_contiguous() and t.dtype == z1.dtype), "gated_add: z, a, f must be [T, d] alike")
    _need((z2 is None) == (f is None), "gated_add: the second sublayer needs its gate")
    _f32v(b1, "b1", d); _f32v(b2, "b2", d)
    fn = _fn("norm", "si_gated_add", [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p])
    _check(fn(_ptr(resid), _ptr(z1), _ptr(b1), _ptr(a), _ptr(z2), _ptr(b2), _ptr(f), _dt(z1), T, d, float(mult), _stream()),
           f"gated_add(hidden={d})")
