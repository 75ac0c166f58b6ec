"""Typed Python entry points of the CUDA kernels (ctypes over the libraries of build.py).

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, shapes), launches on torch's current stream and raises `KernelError` if the
kernel refuses the sizes or the launch fails.  Nothing here computes on the host, and
nothing falls back to a library when the extension is missing.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_float, c_longlong, c_void_p

import torch

from . import build as _build

ERR_UNSUPPORTED = 100001
PAGE = 64            # tokens per cache page; must equal OE_PAGE of common.cuh
MAX_HEAD_DIM = 256   # the largest head size the attention kernels take; must equal MAX_HD of attention.cu


class KernelError(RuntimeError):
    pass


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("oracle_engine_b200 needs a CUDA device (B200, sm_100a): there is no CPU path")


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_SIGNATURES = {
    "elementwise": {
        "oe_embed_gather": [_P, _P, _P, _I, _I, _I, _P, _P],
        "oe_rmsnorm": [_P, _P, _P, _I, _I, _F, _P],
        "oe_rope_kv_write": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "oe_swiglu": [_P, _P, _I, _I, _P],
        "oe_gather_rows_f32": [_P, _P, _P, _I, _I, _P],
    },
    "gemm_simple": {
        "oe_gemm_simple": [_P, _P, _P, _I, _I, _I, _L, _L, _I, _P],
    },
    "attention": {
        "oe_attn_paged": [_P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    },
    "rowwise": {
        "oe_cast_rows_bf16": [_P, _P, _L, _P],
        "oe_rmsnorm_add": [_P, _P, _P, _I, _I, _F, _F, _I, _P, _P],
        "oe_relu2": [_P, _L, _P],
        "oe_tanh_rows": [_P, _P, _L, _P],
        "oe_head_gate": [_P, _P, _L, _P, _L, _P, _I, _I, _I, _I, _I, _I, _F, _P],
        "oe_rot_norm_kv_write": [_P, _L, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P],
        "oe_scaled_add": [_P, _P, _P, _P, _F, _F, _F, _L, _I, _P],
    },
    "attention_split": {
        "oe_rope_split_kv_write": [_P, _L, _P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "oe_attn_split": [_P, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P, _P, _P],
    },
    "attention_prep": {
        "oe_qkv_norm_rot_write": [_P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _F, _P, _P, _I, _P, _P, _I, _P, _I, _P, _P,
                                  _I, _I, _I, _I, _I, _P],
        "oe_unrotate_heads": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    },
    "tokenwise": {
        "oe_dyt_norm": [_P, _P, _P, _P, _F, _L, _I, _P],
        "oe_pair_embed": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _F, _P, _P],
        "oe_prev_token_update": [_P, _P, _P, _P, _I, _P],
        "oe_pass_entry_add": [_P, _P, _P, _L, _I, _P],
        "oe_scale_rows": [_P, _L, _F, _P],
    },
    "general_delta": {
        "oe_gdelta_padded_dk": [_I],
        "oe_gdelta_prepare": [_P, _P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _F, _P, _I, _I, _I, _P],
        "oe_gdelta_scan": [_P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _P],
    },
    "retention": {
        "oe_retention_scan": [_P, _P, _P, _L, _I, _I, _I, _P, _P, _I, _F, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "oe_retention_chunks": [_P, _P, _P, _L, _I, _I, _I, _P, _P, _I, _F, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P],
    },
    "moe": {
        "oe_moe_route": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _I, _P, _P],
        "oe_moe_dense_act": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P],
    },
    "stream": {
        "oe_group_rmsnorm": [_P, _P, _L, _P, _I, _I, _I, _F, _P],
        "oe_group_rmsnorm_add": [_P, _P, _P, _I, _I, _I, _F, _F, _I, _P, _P],
        "oe_poly_norm": [_P, _P, _L, _P, _I, _I, _F, _P],
        "oe_side_gate": [_P, _P, _P, _L, _I, _I, _P, _P, _I, _I, _P],
        "oe_depth_average": [_P, _P, _L, _P, _I, _L, _P],
    },
    "gla": {
        "oe_gla_scan": [_P, _P, _P, _P, _P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _I, _F, _F, _P],
        "oe_gla_scan_segments": [_P, _P, _P, _P, _P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _I, _F, _F, _I, _I, _P, _P, _P],
    },
    "attention_latent": {
        "oe_latent_write": [_P, _L, _P, _F, _P, _L, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "oe_attn_latent": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _P],
        "oe_head_matmul": [_P, _L, _L, _P, _L, _L, _P, _I, _I, _I, _I, _P],
    },
    "recurrent": {
        "oe_short_conv_prepare": [_P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
        "oe_conv_state_update": [_P, _P, _I, _I, _I, _P, _P, _I, _P],
        "oe_delta_rule_scan": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "oe_token_shift_mix": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P],
        "oe_last_rows_to_state": [_P, _P, _I, _P, _P, _I, _P],
        "oe_decay_scan": [_P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _I, _I, _I, _P],
    },
    "sampling": {
        "oe_argmax_rows": [_P, _P, _I, _I, _P],
        "oe_argmax_rows_wide": [_P, _P, _P, _P, _I, _I, _P],
        "oe_sample_rows": [_P, _P, _P, _I, _I, _F, _I, _F, _F, _I, _P, _P, _P, _P, _I, _I, _P],
    },
}
_TYPED = {"oe_embed_gather", "oe_rmsnorm", "oe_rope_kv_write", "oe_swiglu", "oe_gemm_simple", "oe_attn_paged",
          "oe_relu2", "oe_tanh_rows", "oe_rot_norm_kv_write", "oe_token_shift_mix", "oe_last_rows_to_state",
          "oe_rope_split_kv_write", "oe_attn_split", "oe_moe_dense_act", "oe_group_rmsnorm", "oe_poly_norm",
          "oe_side_gate", "oe_latent_write", "oe_attn_latent", "oe_head_matmul", "oe_dyt_norm", "oe_pair_embed",
          "oe_qkv_norm_rot_write", "oe_unrotate_heads"}
_fn_cache: dict[str, object] = {}


def _fn(lib: str, name: str, dtype=None, in_dtype=None):
    full = f"{name}_{_SUFFIX[dtype]}" if name in _TYPED else name
    if in_dtype is not None:                       # kernels typed by their input and their output
        full = f"{name}_{_SUFFIX[in_dtype]}_{_SUFFIX[dtype]}"
    f = _fn_cache.get(full)
    if f is None:
        f = getattr(_build.load(lib), full)
        f.argtypes = _SIGNATURES[lib][name]
        f.restype = c_int
        _fn_cache[full] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  torch.cuda.current_stream() builds a Python object on
    every call (about 17 us); the raw query is what a kernel launch per few microseconds needs."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = [0]          # kernels launched through this module (or captured into a graph)
# ORACLE_SYNC_LAUNCHES=1: the host waits for every kernel right after its launch and names, on standard error, the
# ones that take longer than a second (with what they were launched for): the way to find a kernel that stands
# still, since with the stream running ahead the host only ever waits in the step's last call.
import os as _os
import sys as _sys
import time as _time
SYNC_LAUNCHES = _os.environ.get("ORACLE_SYNC_LAUNCHES", "") not in ("", "0")
OBSERVER = [None]       # engine/profile.py: an object whose mark(what, detail) hears of every launch


def _check(code: int, what: str, detail=None) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        if OBSERVER[0] is not None:
            OBSERVER[0].mark(what, detail)
        if SYNC_LAUNCHES and not torch.cuda.is_current_stream_capturing():
            t0 = _time.time()
            print(f"[launch] {what} {detail if detail is not None else ''}", file=_sys.stderr, flush=True)
            torch.cuda.synchronize()
            if _time.time() - t0 > 1.0:
                print(f"[launch] {what} took {_time.time() - t0:.1f} s", file=_sys.stderr, flush=True)
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: sizes outside what this kernel takes")
    raise KernelError(f"{what}: CUDA error {code} at launch ({torch.cuda.get_device_name()})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ----------------------------------------------------------------------------------------

def embed_gather(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, err: torch.Tensor | None) -> None:
    """x[t] = table[ids[t]] as float32; ids outside the table set err[0] = 1 and give zeros."""
    _dev(x, table, ids, err)
    _i32(ids, "ids")
    n, D = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or not table.is_contiguous() or table.shape[1] != D:
        raise KernelError("embed_gather: x must be float32 [n, D] and table [V, D], contiguous")
    if ids.numel() < n:
        raise KernelError("embed_gather: fewer ids than rows")
    _check(_fn("elementwise", "oe_embed_gather", table.dtype)(
        _ptr(x), _ptr(table), _ptr(ids), n, D, table.shape[0], _ptr(err), _stream()), "embed_gather")


def rmsnorm(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float) -> None:
    """y = (x / sqrt(mean(x^2) + eps)) * w, x float32 [rows, D], w float32 [D]."""
    _dev(y, x, w)
    rows, D = x.shape
    if x.dtype != torch.float32 or w.dtype != torch.float32 or w.numel() != D or y.shape != x.shape:
        raise KernelError("rmsnorm: x and w must be float32, y of x's shape")
    if not (x.is_contiguous() and y.is_contiguous() and w.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    _check(_fn("elementwise", "oe_rmsnorm", y.dtype)(_ptr(y), _ptr(x), _ptr(w), rows, D, float(eps), _stream()),
           "rmsnorm")


def rope_kv_write(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
                  cache: torch.Tensor | None, tables: torch.Tensor, tok_seq: torch.Tensor,
                  tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, has_kv: bool) -> None:
    """Rotates q (in place) and k at each token's position and writes k, v to the paged cache.

    qkv [T, (H + 2 KVH) hd] (or [T, H hd] when has_kv is false); cos/sin float32
    [max_pos, hd/2] or None for no rotation; cache one entry [pages, 2, KVH, PAGE, hd];
    tables int32 [B, max_pages]; tok_seq / tok_pos int32 [T] (tok_seq < 0: padding row)."""
    _dev(qkv, cos, sin, cache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    T = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError(f"rope_kv_write: qkv must be [T, {width}]")
    rotate = cos is not None
    if rotate and (cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2 or not cos.is_contiguous()
                   or sin.shape != cos.shape or not sin.is_contiguous()):
        raise KernelError("rope_kv_write: cos/sin must be float32 [max_pos, head_dim/2]")
    if has_kv:
        if cache is None or cache.dtype != qkv.dtype or not cache.is_contiguous() or \
                tuple(cache.shape[1:]) != (2, n_kv_heads, PAGE, head_dim):
            raise KernelError("rope_kv_write: cache entry must be [pages, 2, KVH, PAGE, head_dim] of qkv's dtype")
    _check(_fn("elementwise", "oe_rope_kv_write", qkv.dtype)(
        _ptr(qkv), qkv.stride(0), _ptr(cos), _ptr(sin), _ptr(cache), _ptr(tables), tables.shape[1],
        _ptr(tok_seq), _ptr(tok_pos), T, n_heads, n_kv_heads, head_dim, int(has_kv), int(rotate), _stream()),
        "rope_kv_write")


def swiglu(out: torch.Tensor, gu: torch.Tensor) -> None:
    """out = silu(gu[:, :FF]) * gu[:, FF:]."""
    _dev(out, gu)
    rows, FF = out.shape
    if gu.shape != (rows, 2 * FF) or gu.dtype != out.dtype or not (gu.is_contiguous() and out.is_contiguous()):
        raise KernelError("swiglu: gu must be [rows, 2 FF] and out [rows, FF], same dtype, contiguous")
    _check(_fn("elementwise", "oe_swiglu", out.dtype)(_ptr(out), _ptr(gu), rows, FF, _stream()), "swiglu")


def gather_rows_f32(out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor) -> None:
    _dev(out, x, rows)
    _i32(rows, "rows")
    if x.dtype != torch.float32 or out.dtype != torch.float32 or not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("gather_rows_f32: float32 contiguous tensors expected")
    _check(_fn("elementwise", "oe_gather_rows_f32")(_ptr(out), _ptr(x), _ptr(rows), out.shape[0], x.shape[1],
                                                    _stream()), "gather_rows_f32")


def gemm_simple(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T on the CUDA cores with float32 accumulation in k order.

    a [M, K] and w [N, K] of one dtype (float32 or bfloat16); out [M, N] of that dtype or
    float32; accumulate needs a float32 out."""
    _dev(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.dtype != w.dtype or not w.is_contiguous():
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows of a and out must be contiguous")
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulate needs a float32 output")
        kind = 2
    elif out.dtype == a.dtype:
        kind = 0
    elif out.dtype == torch.float32:
        kind = 1
    else:
        raise KernelError("gemm: output must have the inputs' dtype or float32")
    _check(_fn("gemm_simple", "oe_gemm_simple", a.dtype)(
        _ptr(out), _ptr(a), _ptr(w), M, N, K, a.stride(0), out.stride(0), kind, _stream()), "gemm_simple")


def attn_paged(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, tables: torch.Tensor,
               tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
               window: int, scale: float, sink: bool = False) -> None:
    """out[t] = attention of token t's query heads over keys (pos-window, pos] of its sequence.

    q [T, >= H hd] (row stride free, e.g. a view of the qkv buffer), out [T, H hd].
    sink: the softmax's denominator gets one added (a key of score 0 without a value)."""
    _dev(out, q, cache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    T = out.shape[0]
    if out.shape[1] != n_heads * head_dim or not out.is_contiguous() or q.stride(1) != 1 or q.dtype != out.dtype:
        raise KernelError("attn_paged: out must be contiguous [T, H hd] and q of its dtype")
    if cache.dtype != out.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (2, n_kv_heads, PAGE, head_dim):
        raise KernelError("attn_paged: cache entry must be [pages, 2, KVH, PAGE, head_dim]")
    _check(_fn("attention", "oe_attn_paged", out.dtype)(
        _ptr(out), _ptr(q), q.stride(0), _ptr(cache), _ptr(tables), tables.shape[1], _ptr(tok_seq), _ptr(tok_pos),
        T, n_heads, n_kv_heads, head_dim, int(window), float(scale), int(bool(sink)), _stream()), "attn_paged")


# ---------------------------------------------------------------------------------------- rowwise.cu

def _f32c(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous float32 tensor")


def cast_rows(y: torch.Tensor, x: torch.Tensor) -> None:
    """y = x (float32) rounded to bfloat16."""
    _dev(y, x)
    _f32c(x, "x")
    if y.dtype != torch.bfloat16 or y.shape != x.shape or not y.is_contiguous():
        raise KernelError("cast_rows: y must be contiguous bfloat16 of x's shape")
    _check(_fn("rowwise", "oe_cast_rows_bf16")(_ptr(y), _ptr(x), x.numel(), _stream()), "cast_rows")


def rmsnorm_add(dst: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, coef: float = 1.0,
                accumulate: bool = True, cast_out: torch.Tensor | None = None) -> None:
    """dst (+)= coef * (y / sqrt(mean(y^2) + eps)) * w; all float32, rows of dst and y correspond.
    accumulate False: dst is written without being read.  cast_out: a contiguous bfloat16 tensor of dst's
    shape that receives the new dst, rounded."""
    _dev(dst, y, w, cast_out)
    if cast_out is not None and (cast_out.dtype != torch.bfloat16 or cast_out.shape != dst.shape
                                 or not cast_out.is_contiguous()):
        raise KernelError("rmsnorm_add: cast_out must be contiguous bfloat16 of dst's shape")
    for t, n in ((dst, "dst"), (y, "y"), (w, "w")):
        _f32c(t, n)
    rows, D = y.shape
    if dst.shape != y.shape or w.numel() != D:
        raise KernelError("rmsnorm_add: dst of y's shape and w of its width expected")
    _check(_fn("rowwise", "oe_rmsnorm_add")(_ptr(dst), _ptr(y), _ptr(w), rows, D, float(eps), float(coef),
                                            int(bool(accumulate)), _ptr(cast_out), _stream()), "rmsnorm_add")


def relu2_(a: torch.Tensor) -> None:
    """a = max(a, 0)^2 in place."""
    _dev(a)
    if not a.is_contiguous() or a.dtype not in _SUFFIX:
        raise KernelError("relu2: a contiguous float32 or bfloat16 tensor expected")
    _check(_fn("rowwise", "oe_relu2", a.dtype)(_ptr(a), a.numel(), _stream()), "relu2")


def tanh_rows(y: torch.Tensor, x: torch.Tensor) -> None:
    """y = tanh(x); x float32, y float32 or bfloat16."""
    _dev(y, x)
    _f32c(x, "x")
    if y.shape != x.shape or not y.is_contiguous() or y.dtype not in _SUFFIX:
        raise KernelError("tanh_rows: y must be contiguous, of x's shape")
    _check(_fn("rowwise", "oe_tanh_rows", y.dtype)(_ptr(y), _ptr(x), x.numel(), _stream()), "tanh_rows")


def head_gate(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor | None, n_heads: int, dv: int,
              norm: bool, act: str, eps: float = 0.0) -> None:
    """out[t, h] = [o[t, h] / sqrt(mean(o[t, h]^2) + eps)] * [w] * act(gate[t, h]) for every head.

    o and gate [T, >= H dv] of one dtype (row strides free), out contiguous [T, H dv]; w None, [dv]
    (shared by the heads) or [H dv], float32; act "sigmoid" or "silu"."""
    _dev(out, o, gate, w)
    T = out.shape[0]
    if out.shape[1] != n_heads * dv or not out.is_contiguous() or o.stride(1) != 1 or gate.stride(1) != 1 \
            or o.dtype != gate.dtype or o.shape[1] < n_heads * dv or gate.shape[1] < n_heads * dv:
        raise KernelError("head_gate: out contiguous [T, H dv]; o and gate of one dtype with at least H dv columns")
    if (o.dtype, out.dtype) not in ((torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                    (torch.bfloat16, torch.bfloat16)):
        raise KernelError(f"head_gate: no kernel for {o.dtype} -> {out.dtype}")
    wmode = 0
    if w is not None:
        _f32c(w, "w")
        wmode = 1 if w.numel() == dv and n_heads * dv != dv else (2 if w.numel() == n_heads * dv else -1)
        if wmode < 0:
            raise KernelError("head_gate: w must hold dv or H dv values")
    _check(_fn("rowwise", "oe_head_gate", out.dtype, o.dtype)(
        _ptr(out), _ptr(o), o.stride(0), _ptr(gate), gate.stride(0), _ptr(w), T, n_heads, dv, int(bool(norm)), wmode,
        {"sigmoid": 0, "silu": 1}[act], float(eps), _stream()), "head_gate")


def rot_norm_kv_write(qk: torch.Tensor, inv_freq: torch.Tensor | None, rot_dims: int, cache: torch.Tensor | None,
                      tables: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int,
                      n_kv_heads: int, head_dim: int, eps: float, has_kv: bool) -> None:
    """Rotates pairs (2i, 2i+1), i < rot_dims/2, of every q and k head by float(pos) * inv_freq[i], divides each head by
    its root mean square (eps inside the root), and writes q back in place, k to the cache's key rows and the k
    as projected to its value rows.  qk [T, >= (H + KVH) hd]; cache [pages, 2, KVH, PAGE, hd]."""
    _dev(qk, inv_freq, cache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    width = (n_heads + (n_kv_heads if has_kv else 0)) * head_dim
    if qk.shape[1] < width or qk.stride(1) != 1:
        raise KernelError(f"rot_norm_kv_write: qk needs at least {width} contiguous columns")
    if rot_dims:
        _f32c(inv_freq, "inv_freq")
        if inv_freq.numel() < rot_dims // 2:
            raise KernelError("rot_norm_kv_write: inv_freq holds fewer values than rotated pairs")
    if has_kv and (cache is None or cache.dtype != qk.dtype or not cache.is_contiguous()
                   or tuple(cache.shape[1:]) != (2, n_kv_heads, PAGE, head_dim)):
        raise KernelError("rot_norm_kv_write: cache entry must be [pages, 2, KVH, PAGE, head_dim] of qk's dtype")
    _check(_fn("rowwise", "oe_rot_norm_kv_write", qk.dtype)(
        _ptr(qk), qk.stride(0), _ptr(inv_freq), int(rot_dims), _ptr(cache), _ptr(tables), tables.shape[1],
        _ptr(tok_seq), _ptr(tok_pos), qk.shape[0], n_heads, n_kv_heads, head_dim, float(eps), int(bool(has_kv)),
        _stream()), "rot_norm_kv_write")


def scaled_add(dst: torch.Tensor, y0: torch.Tensor, vec: torch.Tensor | None = None, mult: float = 1.0,
               c0: float = 1.0, y1: torch.Tensor | None = None, c1: float = 0.0) -> None:
    """dst += mult * vec * (c0 y0 + c1 y1); all float32 and contiguous, vec one value per column (or None: ones)."""
    _dev(dst, y0, y1, vec)
    for t, n in ((dst, "dst"), (y0, "y0")) + (((y1, "y1"),) if y1 is not None else ()) + \
            (((vec, "vec"),) if vec is not None else ()):
        _f32c(t, n)
    rows, D = dst.shape
    if y0.shape != dst.shape or (y1 is not None and y1.shape != dst.shape) or (vec is not None and vec.numel() != D):
        raise KernelError("scaled_add: y0 and y1 of dst's shape and vec of its width expected")
    _check(_fn("rowwise", "oe_scaled_add")(_ptr(dst), _ptr(y0), _ptr(y1), _ptr(vec), float(mult), float(c0), float(c1),
                                           rows, D, _stream()), "scaled_add")


# ---------------------------------------------------------------------------------------- attention_split.cu

def _split_cache_ok(kcache, vcache, dtype, G, dk, dv) -> bool:
    return (kcache is not None and vcache is not None and kcache.dtype == dtype and vcache.dtype == dtype
            and kcache.is_contiguous() and vcache.is_contiguous()
            and tuple(kcache.shape[1:]) == (G, PAGE, dk) and tuple(vcache.shape[1:]) == (G, PAGE, dv))


def rope_split_kv_write(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, rot_dims: int,
                        kcache: torch.Tensor | None, vcache: torch.Tensor | None, tables: torch.Tensor,
                        tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, dk: int, dv: int,
                        has_kv: bool = True) -> None:
    """Turns the first rot_dims dimensions of every q head (in place) and k head (dimension i < rot_dims/2 with
    i + rot_dims/2) by the token's position, and writes k to the key tensor and v to the value tensor of the cache.

    qkv [T, >= H dk + G dk + G dv]; cos/sin float32 [positions, rot_dims/2]; kcache [pages, G, PAGE, dk],
    vcache [pages, G, PAGE, dv] of qkv's dtype; tok_seq < 0 marks a padding row."""
    _dev(qkv, cos, sin, kcache, vcache, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    width = n_heads * dk + (n_kv_heads * (dk + dv) if has_kv else 0)
    if qkv.shape[1] < width or qkv.stride(1) != 1:
        raise KernelError(f"rope_split_kv_write: qkv needs at least {width} contiguous columns")
    if rot_dims:
        _f32c(cos, "cos")
        _f32c(sin, "sin")
        if rot_dims % 2 or rot_dims > dk or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
            raise KernelError("rope_split_kv_write: cos/sin must be [positions, rot_dims/2], rot_dims even and <= dk")
    if has_kv and not _split_cache_ok(kcache, vcache, qkv.dtype, n_kv_heads, dk, dv):
        raise KernelError("rope_split_kv_write: the cache must be [pages, G, PAGE, dk] and [pages, G, PAGE, dv] of qkv's dtype")
    _check(_fn("attention_split", "oe_rope_split_kv_write", qkv.dtype)(
        _ptr(qkv), qkv.stride(0), _ptr(cos), _ptr(sin), int(rot_dims), _ptr(kcache), _ptr(vcache), _ptr(tables),
        tables.shape[1], _ptr(tok_seq), _ptr(tok_pos), qkv.shape[0], n_heads, n_kv_heads, dk, dv, int(bool(has_kv)),
        _stream()), "rope_split_kv_write")


def _unrotate_tables(unrotate, dv: int, what: str):
    """(cos, sin) checked: float32 [positions, dv/2] on the device, dv even; (None, None) if there is nothing to turn."""
    if unrotate is None:
        return None, None
    uc, us = unrotate
    _dev(uc, us)
    _f32c(uc, "cos")
    _f32c(us, "sin")
    if dv % 2 or uc.dim() != 2 or uc.shape[1] != dv // 2 or us.shape != uc.shape:
        raise KernelError(f"{what}: the tables of the turn back must be [positions, dv/2], dv even")
    return uc, us


def attn_split(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, tables: torch.Tensor,
               tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int, n_kv_heads: int, dk: int, dv: int,
               window: int, scale: float, cap: float = 0.0, sinks: torch.Tensor | None = None, unrotate=None) -> None:
    """out[t] = softmax attention of token t's query heads over the keys (pos - window, pos] of its sequence, with
    s <- cap tanh(s / cap) when cap > 0.  q [T, >= H dk] (row stride free), out contiguous [T, H dv].  sinks (float32
    [H] or None): exp(sinks[h]) is one more term of head h's denominator, without key or value.  unrotate ((cos, sin)
    float32 [positions, dv/2] or None): every head's result is turned back by its query's position before it is stored."""
    _dev(out, q, kcache, vcache, tables, tok_seq, tok_pos, sinks)
    uc, us = _unrotate_tables(unrotate, dv, "attn_split")
    if sinks is not None:
        _f32c(sinks, "sinks")
        if sinks.numel() != n_heads:
            raise KernelError("attn_split: sinks must hold one value per query head")
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    if out.shape[1] != n_heads * dv or not out.is_contiguous() or q.stride(1) != 1 or q.dtype != out.dtype \
            or q.shape[1] < n_heads * dk:
        raise KernelError("attn_split: out must be contiguous [T, H dv] and q of its dtype with at least H dk columns")
    if not _split_cache_ok(kcache, vcache, out.dtype, n_kv_heads, dk, dv):
        raise KernelError("attn_split: the cache must be [pages, G, PAGE, dk] and [pages, G, PAGE, dv] of out's dtype")
    _check(_fn("attention_split", "oe_attn_split", out.dtype)(
        _ptr(out), _ptr(q), q.stride(0), _ptr(kcache), _ptr(vcache), _ptr(tables), tables.shape[1], _ptr(tok_seq),
        _ptr(tok_pos), out.shape[0], n_heads, n_kv_heads, dk, dv, int(window), float(scale), float(cap or 0.0),
        _ptr(sinks), _ptr(uc), _ptr(us), _stream()), "attn_split")


# ---------------------------------------------------------------------------------------- attention_prep.cu

def qkv_norm_rot_write(q_out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, proj: torch.Tensor,
                       biases, norm_weights, eps: float, key_tables, rot_dims: int, value_tables, value_norm: bool,
                       tables: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int,
                       n_kv_heads: int, dk: int, dv: int) -> None:
    """From the float32 projection rows proj [T, >= H dk + G dk + G dv] = [q | k | v]: adds `biases` (three float32
    vectors or None), divides every q and k head by its root mean square and multiplies by `norm_weights` (two
    float32 vectors [dk], or None: no norm), turns their first rot_dims dimensions by the position (halves paired;
    key_tables = (cos, sin) float32 [positions, rot_dims/2] or None), divides every v head by its root mean square
    when value_norm, and turns all dv dimensions of v by the position (value_tables = (cos, sin) [positions, dv/2] or
    None).  q goes to q_out [T, H dk] (contiguous, the cache's dtype), k and v to the token's rows of the cache."""
    qb, kb, vb = biases if biases is not None else (None, None, None)
    qw, kw = norm_weights if norm_weights is not None else (None, None)
    ck, sk = key_tables if key_tables is not None and rot_dims else (None, None)
    cv, sv = value_tables if value_tables is not None else (None, None)
    _dev(q_out, kcache, vcache, proj, qb, kb, vb, qw, kw, ck, sk, cv, sv, tables, tok_seq, tok_pos)
    for t, n in ((tables, "tables"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        _i32(t, n)
    T = proj.shape[0]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < n_heads * dk + n_kv_heads * (dk + dv):
        raise KernelError("qkv_norm_rot_write: proj must be float32 rows of at least H dk + G (dk + dv) values")
    if tuple(q_out.shape) != (T, n_heads * dk) or not q_out.is_contiguous() or q_out.dtype not in _SUFFIX:
        raise KernelError("qkv_norm_rot_write: q_out must be contiguous [T, H dk]")
    if not _split_cache_ok(kcache, vcache, q_out.dtype, n_kv_heads, dk, dv):
        raise KernelError("qkv_norm_rot_write: the cache must be [pages, G, PAGE, dk] and [pages, G, PAGE, dv] of q_out's dtype")
    for t, n, size in ((qb, "q bias", n_heads * dk), (kb, "k bias", n_kv_heads * dk), (vb, "v bias", n_kv_heads * dv),
                       (qw, "q norm weight", dk), (kw, "k norm weight", dk)):
        if t is not None:
            _f32c(t, n)
            if t.numel() != size:
                raise KernelError(f"qkv_norm_rot_write: {n} must hold {size} values")
    if (qw is None) != (kw is None):
        raise KernelError("qkv_norm_rot_write: q and k are normed together or not at all")
    if ck is not None:
        _f32c(ck, "cos")
        _f32c(sk, "sin")
        if rot_dims % 2 or rot_dims > dk or ck.shape[1] != rot_dims // 2 or sk.shape != ck.shape:
            raise KernelError("qkv_norm_rot_write: key tables must be [positions, rot_dims/2], rot_dims even and <= dk")
    if cv is not None:
        _f32c(cv, "value cos")
        _f32c(sv, "value sin")
        if dv % 2 or cv.shape[1] != dv // 2 or sv.shape != cv.shape:
            raise KernelError("qkv_norm_rot_write: value tables must be [positions, dv/2], dv even")
    _check(_fn("attention_prep", "oe_qkv_norm_rot_write", q_out.dtype)(
        _ptr(q_out), _ptr(kcache), _ptr(vcache), _ptr(proj), proj.stride(0), _ptr(qb), _ptr(kb), _ptr(vb), _ptr(qw),
        _ptr(kw), float(eps), _ptr(ck), _ptr(sk), int(rot_dims if ck is not None else 0), _ptr(cv), _ptr(sv),
        int(bool(value_norm)), _ptr(tables), tables.shape[1], _ptr(tok_seq), _ptr(tok_pos), T, n_heads, n_kv_heads, dk, dv,
        _stream()), "qkv_norm_rot_write")


def unrotate_heads(o: torch.Tensor, value_tables, tok_seq: torch.Tensor, tok_pos: torch.Tensor, n_heads: int,
                   dv: int) -> None:
    """Every head of o [T, H dv] (contiguous) turned back by its token's position, in place: the pair (m, m + dv/2)
    by minus the angle whose cosine and sine value_tables = (cos, sin) float32 [positions, dv/2] hold."""
    cv, sv = value_tables
    _dev(o, cv, sv, tok_seq, tok_pos)
    _i32(tok_seq, "tok_seq")
    _i32(tok_pos, "tok_pos")
    _f32c(cv, "value cos")
    _f32c(sv, "value sin")
    if o.dtype not in _SUFFIX or not o.is_contiguous() or o.shape[1] != n_heads * dv or dv % 2 \
            or cv.shape[1] != dv // 2 or sv.shape != cv.shape:
        raise KernelError("unrotate_heads: o contiguous [T, H dv], dv even, tables [positions, dv/2]")
    _check(_fn("attention_prep", "oe_unrotate_heads", o.dtype)(
        _ptr(o), _ptr(cv), _ptr(sv), _ptr(tok_seq), _ptr(tok_pos), o.shape[0], n_heads, dv, _stream()), "unrotate_heads")


# ---------------------------------------------------------------------------------------- tokenwise.cu

def dyt_norm(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: float) -> None:
    """y = tanh(alpha x) * w + b; x float32 [rows, D], w and b float32 [D], y float32 or bfloat16 of x's shape."""
    _dev(y, x, w, b)
    for t, n in ((x, "x"), (w, "w"), (b, "b")):
        _f32c(t, n)
    D = x.shape[-1]
    if y.shape != x.shape or not y.is_contiguous() or y.dtype not in _SUFFIX or w.numel() != D or b.numel() != D:
        raise KernelError("dyt_norm: y contiguous of x's shape, w and b one value per column")
    _check(_fn("tokenwise", "oe_dyt_norm", y.dtype)(_ptr(y), _ptr(x), _ptr(w), _ptr(b), float(alpha), x.numel() // D, D,
                                                    _stream()), "dyt_norm")


def pair_embed(x: torch.Tensor, table: torch.Tensor, pair: torch.Tensor | None, ctx, prev: torch.Tensor | None,
               buckets: int, mul_prev: int, mul_cur: int, scale: float, err: torch.Tensor | None) -> None:
    """x[t] = table[id_t] * scale + pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] as float32, row `buckets` of
    `pair` for a sequence's first token; the token before a step's first one comes from prev [slots] int32.  pair
    None: the scaled table row alone.  Padding rows get zeros; an id outside the table sets err[0] = 1."""
    _dev(x, table, pair, prev, err, ctx.token_ids)
    n, D = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or not table.is_contiguous() or table.shape[1] != D:
        raise KernelError("pair_embed: x must be float32 [n, D] and table [V, D], contiguous")
    if pair is not None:
        if pair.dtype != table.dtype or not pair.is_contiguous() or tuple(pair.shape) != (buckets + 1, D):
            raise KernelError("pair_embed: the pair table must be [buckets + 1, D] of the table's dtype")
        if prev is None or prev.dtype != torch.int32 or not prev.is_contiguous():
            raise KernelError("pair_embed: prev must be a contiguous int32 tensor, one value per slot")
    if ctx.token_ids.numel() < n or ctx.tok_seq.numel() < n:
        raise KernelError("pair_embed: fewer ids than rows")
    _check(_fn("tokenwise", "oe_pair_embed", table.dtype)(
        _ptr(x), _ptr(table), _ptr(pair), _ptr(ctx.token_ids), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.cu_q),
        _ptr(ctx.seq_slot), _ptr(prev), n, D, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), float(scale),
        _ptr(err), _stream()), "pair_embed")


def prev_token_update(prev: torch.Tensor, ctx) -> None:
    """prev[slot of sequence b] = the last token sequence b brings in this step."""
    _dev(prev, ctx.token_ids)
    if prev.dtype != torch.int32 or not prev.is_contiguous():
        raise KernelError("prev_token_update: prev must be a contiguous int32 tensor")
    _check(_fn("tokenwise", "oe_prev_token_update")(_ptr(prev), _ptr(ctx.token_ids), _ptr(ctx.cu_q), _ptr(ctx.seq_slot),
                                                    ctx.n_seqs, _stream()), "prev_token_update")


def pass_entry_add(x: torch.Tensor, e: torch.Tensor | None, s: torch.Tensor) -> None:
    """x += e + s; x and e float32 [rows, D] (e may be None), s float32 [D]."""
    _dev(x, e, s)
    _f32c(x, "x")
    _f32c(s, "s")
    if e is not None:
        _f32c(e, "e")
        if e.shape != x.shape:
            raise KernelError("pass_entry_add: e must have x's shape")
    if s.numel() != x.shape[-1]:
        raise KernelError("pass_entry_add: s must hold one value per column")
    D = x.shape[-1]
    _check(_fn("tokenwise", "oe_pass_entry_add")(_ptr(x), _ptr(e), _ptr(s), x.numel() // D, D, _stream()), "pass_entry_add")


def scale_rows(x: torch.Tensor, s: float) -> None:
    """x *= s; x float32, contiguous."""
    _dev(x)
    _f32c(x, "x")
    _check(_fn("tokenwise", "oe_scale_rows")(_ptr(x), x.numel(), float(s), _stream()), "scale_rows")


# ---------------------------------------------------------------------------------------- general_delta.cu

def gdelta_padded_dk(dk: int) -> int:
    """The number of key channels a packed row of gdelta_prepare holds per vector (dk rounded up), or -1."""
    return int(_fn("general_delta", "oe_gdelta_padded_dk")(int(dk)))


def gdelta_prepare(packed: torch.Tensor, proj: torch.Tensor, off_r: int, off_k: int, off_a: int, off_z1: int, rank: int,
                   w2: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor | None, decay_coef: float, tok_seq: torch.Tensor,
                   heads: int, dk: int) -> None:
    """The vectors a generalized delta rule reads, from float32 projection rows: per (token, head)
    [w | u | a u | k | r w] (each padded to gdelta_padded_dk(dk) values), c1 = sum r a u, c2 = r . k, with
    w = exp(-decay_coef sigmoid(w2 tanh(z1) + w0)), a = sigmoid(za + a_bias), u = k / sqrt(|k|^2 + 1e-6)."""
    _dev(packed, proj, w2, w0, a_bias, tok_seq)
    _i32(tok_seq, "tok_seq")
    for t, n in ((packed, "packed"), (w2, "w2"), (w0, "w0")):
        _f32c(t, n)
    T = proj.shape[0]
    dkp = gdelta_padded_dk(dk)
    if proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelError("gdelta_prepare: proj must be float32 rows")
    if dkp < 0 or tuple(packed.shape) != (T, heads, 5 * dkp + 4) or tuple(w2.shape) != (heads * dk, rank) \
            or w0.numel() != heads * dk or (a_bias is not None and a_bias.numel() != heads * dk):
        raise KernelError("gdelta_prepare: shapes do not agree")
    for off, n in ((off_r, heads * dk), (off_k, heads * dk), (off_a, heads * dk), (off_z1, rank)):
        if off < 0 or off + n > proj.shape[1]:
            raise KernelError("gdelta_prepare: a column range lies outside the projection row")
    if a_bias is not None:
        _f32c(a_bias, "a_bias")
    _check(_fn("general_delta", "oe_gdelta_prepare")(
        _ptr(packed), _ptr(proj), proj.stride(0), off_r, off_k, off_a, off_z1, rank, _ptr(w2), _ptr(w0), _ptr(a_bias),
        float(decay_coef), _ptr(tok_seq), T, heads, dk, _stream()), "gdelta_prepare")


def gdelta_scan(o: torch.Tensor, state: torch.Tensor, packed: torch.Tensor, v: torch.Tensor, ctx, heads: int, dk: int,
                dv: int) -> None:
    """S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r for every token of the step, in order, per sequence and head.
    o float32 [T, H dv] contiguous; state float32 [slots, H, dk, dv]; packed as gdelta_prepare left it; v float32
    [T, H dv] (a view of the projection rows; row stride free)."""
    _dev(o, state, packed, v)
    for t, n in ((o, "o"), (state, "state"), (packed, "packed")):
        _f32c(t, n)
    T = o.shape[0]
    dkp = gdelta_padded_dk(dk)
    if dkp < 0 or tuple(o.shape) != (T, heads * dv) or tuple(state.shape[1:]) != (heads, dk, dv) \
            or tuple(packed.shape) != (T, heads, 5 * dkp + 4) or v.dtype != torch.float32 or v.stride(1) != 1 \
            or tuple(v.shape) != (T, heads * dv):
        raise KernelError("gdelta_scan: shapes do not agree")
    _check(_fn("general_delta", "oe_gdelta_scan")(
        _ptr(o), _ptr(state), _ptr(packed), _ptr(v), v.stride(0), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), ctx.n_seqs, heads, dk,
        dv, _stream()), "gdelta_scan")


# ---------------------------------------------------------------------------------------- retention.cu

def retention_scan(o: torch.Tensor, state: torch.Tensor, proj: torch.Tensor, off_q: int, off_k: int, off_v: int,
                   cos: torch.Tensor | None, sin: torch.Tensor | None, rot_dims: int, k_scale: float,
                   decay: torch.Tensor, ctx, heads: int, dk: int, dv: int, scratch: torch.Tensor | None = None) -> None:
    """Per sequence and head, over the step's tokens in order: S <- decay_h S + k v^T; o = S^T q, with q and k
    turned by the token's position (first rot_dims dimensions, halves paired) and k times k_scale.  proj float32
    [T, >= ...] holds q at column off_q (H dk values), k at off_k (H dk), v at off_v (H dv); state float32
    [slots, H, dk, dv] is read and written; o float32 [T, H dv].  scratch: float32 room for retention_scratch(...)
    values; with it the chunked form runs (a sequence's tokens 32 at a time, the same sums in another order, for
    prompts; it turns and scales q and k in place in proj), without it the tokens go one by one."""
    _dev(o, state, proj, cos, sin, decay)
    for t, n in ((o, "o"), (state, "state"), (decay, "decay")):
        _f32c(t, n)
    T = proj.shape[0]
    if proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelError("retention_scan: proj must be float32 with contiguous rows")
    if tuple(state.shape[1:]) != (heads, dk, dv) or tuple(o.shape) != (T, heads * dv) or decay.numel() != heads \
            or max(off_q + heads * dk, off_k + heads * dk, off_v + heads * dv) > proj.shape[1]:
        raise KernelError("retention_scan: shapes do not agree")
    if rot_dims:
        _f32c(cos, "cos")
        _f32c(sin, "sin")
        if rot_dims % 2 or rot_dims > dk or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
            raise KernelError("retention_scan: cos/sin must be [positions, rot_dims/2], rot_dims even and <= dk")
    if scratch is not None:
        _f32c(scratch, "scratch")
        max_chunks = scratch.numel() // (heads * dk * dv)
        if max_chunks < T // RETENTION_CHUNK + ctx.n_seqs:
            raise KernelError("retention_scan: the scratch is smaller than retention_scratch(...) values")
        _check(_fn("retention", "oe_retention_chunks")(
            _ptr(o), _ptr(state), _ptr(proj), proj.stride(0), int(off_q), int(off_k), int(off_v), _ptr(cos), _ptr(sin),
            int(rot_dims), float(k_scale), _ptr(decay), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), _ptr(ctx.tok_seq),
            _ptr(ctx.tok_pos), T, ctx.n_seqs, heads, dk, dv, _ptr(scratch), max_chunks, _stream()), "retention_chunks")
        LAUNCHES[0] += 3
        return
    _check(_fn("retention", "oe_retention_scan")(
        _ptr(o), _ptr(state), _ptr(proj), proj.stride(0), int(off_q), int(off_k), int(off_v), _ptr(cos), _ptr(sin),
        int(rot_dims), float(k_scale), _ptr(decay), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), _ptr(ctx.tok_pos), ctx.n_seqs,
        heads, dk, dv, _stream()), "retention_scan")


RETENTION_CHUNK = 32      # tokens per chunk of the chunked retention; must equal CC of retention.cu


def retention_scratch(n_tokens: int, n_seqs: int, heads: int, dk: int, dv: int) -> int:
    """How many float32 values the chunked retention needs as scratch: a state per chunk and head."""
    return (n_tokens // RETENTION_CHUNK + n_seqs) * heads * dk * dv


# ---------------------------------------------------------------------------------------- moe.cu

def moe_route(z: torch.Tensor, n_experts: int, top: int, has_gate, dense: torch.Tensor, tok_seq: torch.Tensor,
              idx: torch.Tensor | None = None, wt: torch.Tensor | None = None, weights: str = "softmax",
              bias: torch.Tensor | None = None) -> None:
    """From router logits z float32 [T, >= E (+ 1)]: dense [T, E (+ 1)] float32 gets each chosen expert's weight
    (zero elsewhere) and, with has_gate, sigmoid of column E in its last column (has_gate "one": the constant 1, a
    shared expert without a gate; z needs no column for it); idx int32 [T, top] and wt float32 [T, top] receive the
    choice itself when given.  weights "softmax": the softmax over the `top` largest logits alone; "sigmoid": each
    chosen expert's own sigmoid(logit), not renormalised.  bias (float32 [E], with "sigmoid" only): the choice is by
    sigmoid(logit) + bias, the weights stay the sigmoids."""
    _dev(z, dense, tok_seq, idx, wt, bias)
    if bias is not None:
        _f32c(bias, "bias")
        if weights != "sigmoid" or bias.numel() != n_experts:
            raise KernelError("moe_route: a choice bias needs sigmoid weights and one value per expert")
    _i32(tok_seq, "tok_seq")
    _f32c(dense, "dense")
    T = z.shape[0]
    W = n_experts + int(bool(has_gate))
    gate = 2 if has_gate == "one" else int(bool(has_gate))
    if weights not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route: weights must be softmax or sigmoid, got {weights!r}")
    if z.dtype != torch.float32 or z.stride(1) != 1 or z.shape[1] < (n_experts if gate == 2 else W) \
            or tuple(dense.shape) != (T, W):
        raise KernelError("moe_route: z float32 [T, >= E (+1)] and dense [T, E (+1)] expected")
    if top > n_experts:
        raise KernelError("moe_route: more experts chosen than there are")
    if idx is not None:
        _i32(idx, "idx")
    if wt is not None:
        _f32c(wt, "wt")
    for t in (idx, wt):
        if t is not None and tuple(t.shape) != (T, top):
            raise KernelError("moe_route: idx and wt must be [T, top]")
    _check(_fn("moe", "oe_moe_route")(_ptr(z), z.stride(0), n_experts, top, gate, int(weights == "sigmoid"), _ptr(idx), _ptr(wt),
                                      _ptr(dense), _ptr(tok_seq), T, _ptr(bias), _stream()), "moe_route")


def moe_dense_act(a: torch.Tensor, gu: torch.Tensor, dense: torch.Tensor, n_experts: int, ff: int,
                  scale_input: bool = False, act: str = "silu", limit: float = 0.0) -> None:
    """a[t, c] = silu(gu[t, c]) * gu[t, F + c] * dense[t, group of c]; the group of column c is c // ff for the
    first n_experts * ff columns and the last column of dense for the rest (the shared expert).  scale_input: the
    weight w = dense[t, group] multiplies the expert's input instead, a = silu(w gu[t, c]) * (w gu[t, F + c]).
    act "clamped": with g = min(gate, limit) and u = clamp(up, -limit, limit), a = g * sigmoid(1.702 g) * (u + 1) * w."""
    _dev(a, gu, dense)
    if act not in ("silu", "clamped") or (act == "clamped" and (scale_input or not limit > 0)):
        raise KernelError("moe_dense_act: act is silu or clamped (with a positive limit, weight on the output)")
    _f32c(dense, "dense")
    T, F = a.shape
    if tuple(gu.shape) != (T, 2 * F) or gu.dtype != a.dtype or not (gu.is_contiguous() and a.is_contiguous()) \
            or dense.shape[0] != T or dense.shape[1] < n_experts or F < n_experts * ff \
            or (F > n_experts * ff and dense.shape[1] != n_experts + 1):
        raise KernelError("moe_dense_act: shapes do not agree")
    _check(_fn("moe", "oe_moe_dense_act", a.dtype)(_ptr(a), _ptr(gu), _ptr(dense), T, F, n_experts, ff, dense.shape[1],
                                                   int(bool(scale_input)), int(act == "clamped"), float(limit),
                                                   _stream()), "moe_dense_act")


# ---------------------------------------------------------------------------------------- stream.cu

def group_rmsnorm(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> None:
    """y = x cut into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), times w;
    x float32 [rows, D], w float32 [D], y float32 or bfloat16."""
    _dev(y, x, w)
    _f32c(w, "w")
    rows, D = x.shape
    if x.dtype != torch.float32 or x.stride(1) != 1 or y.shape != x.shape or not y.is_contiguous() or w.numel() != D \
            or groups < 1 or D % groups:
        raise KernelError("group_rmsnorm: x float32 (row stride free), y contiguous of x's shape, w [D], D a multiple of groups")
    _check(_fn("stream", "oe_group_rmsnorm", y.dtype)(_ptr(y), _ptr(x), x.stride(0), _ptr(w), rows, D, int(groups), float(eps),
                                                      _stream()), "group_rmsnorm")


def group_rmsnorm_add(dst: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, groups: int, coef: float = 1.0,
                      accumulate: bool = True, cast: torch.Tensor | None = None) -> None:
    """dst (+)= coef * (the grouped norm of y) * w, all float32; cast (bfloat16, dst's shape) also receives the new dst."""
    _dev(dst, y, w, cast)
    for t, n in ((dst, "dst"), (y, "y"), (w, "w")):
        _f32c(t, n)
    rows, D = y.shape
    if dst.shape != y.shape or w.numel() != D or groups < 1 or D % groups:
        raise KernelError("group_rmsnorm_add: dst of y's shape, w [D], D a multiple of groups")
    if cast is not None and (cast.dtype != torch.bfloat16 or cast.shape != dst.shape or not cast.is_contiguous()):
        raise KernelError("group_rmsnorm_add: cast must be a contiguous bfloat16 tensor of dst's shape")
    _check(_fn("stream", "oe_group_rmsnorm_add")(_ptr(dst), _ptr(y), _ptr(w), rows, D, int(groups), float(eps), float(coef),
                                                 int(bool(accumulate)), _ptr(cast), _stream()), "group_rmsnorm_add")


def poly_norm(out: torch.Tensor, z: torch.Tensor, coef: torch.Tensor, eps: float) -> None:
    """out = a R(z) + b R(z^2) + c R(z^3) + e per row with R(u) = u / sqrt(mean(u^2) + eps) and (a, b, c, e) = coef
    (float32 [4] on the device); z float32 [rows, F] (row stride free), out contiguous float32 or bfloat16."""
    _dev(out, z, coef)
    _f32c(coef, "coef")
    rows, F = out.shape
    if z.dtype != torch.float32 or z.shape != out.shape or z.stride(1) != 1 or not out.is_contiguous() or coef.numel() != 4:
        raise KernelError("poly_norm: z float32 [rows, F], out contiguous of that shape, coef [4]")
    _check(_fn("stream", "oe_poly_norm", out.dtype)(_ptr(out), _ptr(z), z.stride(0), _ptr(coef), rows, F, float(eps),
                                                    _stream()), "poly_norm")


def side_gate(g: torch.Tensor, u: torch.Tensor, table: torch.Tensor, offset: int, token_ids: torch.Tensor,
              tok_seq: torch.Tensor) -> None:
    """g[t, j] = gelu_tanh(u[t, j]) * table[token_ids[t], offset + j]; u float32 [T, dim] contiguous, g and table of
    one dtype; rows of padding tokens and ids outside the table give zeros."""
    _dev(g, u, table, token_ids, tok_seq)
    _i32(token_ids, "token_ids")
    _i32(tok_seq, "tok_seq")
    _f32c(u, "u")
    T, dim = u.shape
    if g.shape != u.shape or not g.is_contiguous() or g.dtype != table.dtype or table.stride(1) != 1 \
            or offset < 0 or offset + dim > table.shape[1] or token_ids.numel() < T or tok_seq.numel() < T:
        raise KernelError("side_gate: g of u's shape and the table's dtype, offset + dim within the table's columns")
    _check(_fn("stream", "oe_side_gate", g.dtype)(_ptr(g), _ptr(u), _ptr(table), table.stride(0), int(offset), dim,
                                                  _ptr(token_ids), _ptr(tok_seq), table.shape[0], T, _stream()), "side_gate")


def depth_average(x: torch.Tensor, hist: torch.Tensor, w: torch.Tensor, n: int) -> None:
    """hist[n] = x; x = sum_{j <= n} w[j] * hist[j] (terms added in order of j); x float32 [T, D], hist float32
    [>= n + 1, T, D], w float32 [>= n + 1]."""
    _dev(x, hist, w)
    for t, name in ((x, "x"), (hist, "hist"), (w, "w")):
        _f32c(t, name)
    if hist.dim() != 3 or tuple(hist.shape[1:]) != tuple(x.shape) or hist.shape[0] <= n or w.numel() <= n or n < 0:
        raise KernelError("depth_average: hist [>= n + 1, T, D], w [>= n + 1]")
    _check(_fn("stream", "oe_depth_average")(_ptr(x), _ptr(hist), hist.stride(0), _ptr(w), int(n), x.numel(), _stream()),
           "depth_average")


# ---------------------------------------------------------------------------------------- gla.cu

def gla_scan(o: torch.Tensor, state: torch.Tensor, proj: torch.Tensor, off_q: int, off_k: int, off_v: int, z: torch.Tensor,
             bias: torch.Tensor, ctx, heads: int, dk: int, dv: int, q_scale: float, tau: float, segments=None) -> None:
    """Per sequence and head, over the step's tokens in order: alpha = sigmoid(z + bias)^(1/tau) [dk];
    S <- diag(alpha) S + k v^T; o = S^T (q * q_scale).  proj float32 rows holding q, k (heads*dk) and v (heads*dv) at
    the given column offsets; z float32 [T, heads*dk]; state float32 [slots, heads, dk, dv]; o float32 [T, heads*dv].
    segments (seg_len, n_seg, seg_state, seg_decay): every sequence's tokens (at most seg_len * n_seg) run as segments
    side by side; the scratch tensors are float32 [n_seqs, n_seg, heads, dk, dv] and [n_seqs, n_seg, heads, dk].  The
    result differs from the one walk by the order of the sums only."""
    _dev(o, state, proj, z, bias)
    for t, n in ((o, "o"), (state, "state"), (bias, "bias")):
        _f32c(t, n)
    T = o.shape[0]
    if proj.dtype != torch.float32 or z.dtype != torch.float32 or proj.stride(1) != 1 or z.stride(1) != 1 \
            or proj.shape[0] < T or z.shape[0] < T or z.shape[1] < heads * dk or o.shape[1] != heads * dv \
            or tuple(state.shape[1:]) != (heads, dk, dv) or bias.numel() != heads * dk \
            or max(off_q, off_k) + heads * dk > proj.shape[1] or off_v + heads * dv > proj.shape[1]:
        raise KernelError("gla_scan: shapes do not agree")
    e = proj.element_size()
    base = proj.data_ptr()
    if segments is not None:
        seg_len, n_seg, seg_state, seg_decay = segments
        _dev(seg_state, seg_decay)
        _f32c(seg_state, "seg_state")
        _f32c(seg_decay, "seg_decay")
        if seg_len < 1 or n_seg < 1 or seg_len * n_seg < int(ctx.max_qlen) \
                or seg_state.numel() < ctx.n_seqs * n_seg * heads * dk * dv or seg_decay.numel() < ctx.n_seqs * n_seg * heads * dk:
            raise KernelError("gla_scan: the segments do not cover the step's longest sequence, or their scratch is too small")
        _check(_fn("gla", "oe_gla_scan_segments")(
            _ptr(o), _ptr(state), base + off_q * e, base + off_k * e, base + off_v * e, proj.stride(0), _ptr(z), z.stride(0),
            _ptr(bias), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), ctx.n_seqs, heads, dk, dv, float(q_scale), 1.0 / float(tau),
            int(seg_len), int(n_seg), _ptr(seg_state), _ptr(seg_decay), _stream()), "gla_scan_segments")
        LAUNCHES[0] += 2
        return
    _check(_fn("gla", "oe_gla_scan")(_ptr(o), _ptr(state), base + off_q * e, base + off_k * e, base + off_v * e,
                                     proj.stride(0), _ptr(z), z.stride(0), _ptr(bias), _ptr(ctx.seq_slot), _ptr(ctx.cu_q),
                                     ctx.n_seqs, heads, dk, dv, float(q_scale), 1.0 / float(tau), _stream()), "gla_scan")


# ---------------------------------------------------------------------------------------- attention_latent.cu

def latent_write(d: torch.Tensor | None, w: torch.Tensor | None, eps: float, q: torch.Tensor, qfull: torch.Tensor,
                 freq: torch.Tensor | None, dims: int, cache: torch.Tensor | None, tables: torch.Tensor, ctx, heads: int,
                 dk: int, r: int, rd: int, write_cache: bool) -> None:
    """Per token: the first r values of d's row, divided by their root mean square and times w, and the last rd
    values with their first `dims` turned in pairs (2i, 2i + 1) by position * freq[i], go to the token's cache row
    [r + rd] (only when write_cache); the last rd dimensions of each of q's heads [dk + rd] are turned the same way
    and written to qfull[t, h, r:].  d float32; q, qfull and cache of one dtype."""
    _dev(d, w, q, qfull, freq, cache, tables)
    T = q.shape[0]
    R = r + rd
    if q.stride(1) != 1 or q.shape[1] < heads * (dk + rd) or tuple(qfull.shape) != (T, heads * R) \
            or not qfull.is_contiguous() or q.dtype != qfull.dtype:
        raise KernelError("latent_write: q [T, >= H (dk + rd)], qfull contiguous [T, H (r + rd)] of q's dtype")
    if write_cache:
        if d is None or w is None or cache is None or d.dtype != torch.float32 or d.stride(1) != 1 or d.shape[1] < R \
                or w.dtype != torch.float32 or w.numel() != r or cache.dtype != q.dtype or not cache.is_contiguous() \
                or tuple(cache.shape[1:]) != (PAGE, R):
            raise KernelError("latent_write: d float32 [T, >= r + rd], w float32 [r], cache [pages, PAGE, r + rd]")
    if dims and (freq is None or freq.dtype != torch.float32 or freq.numel() < dims // 2):
        raise KernelError("latent_write: freq float32 [dims / 2]")
    _check(_fn("attention_latent", "oe_latent_write", q.dtype)(
        _ptr(d), 0 if d is None else d.stride(0), _ptr(w), float(eps), _ptr(q), q.stride(0), _ptr(qfull), _ptr(freq),
        int(dims), _ptr(cache), _ptr(tables), tables.shape[1], _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), T, heads, dk, r, rd,
        int(bool(write_cache)), _stream()), "latent_write")


def attn_latent(out: torch.Tensor, qfull: torch.Tensor, cache: torch.Tensor, tables: torch.Tensor, ctx, heads: int, r: int,
                rd: int, scale: float) -> None:
    """out[t, h] = sum_j p_j c_j over the keys j <= pos of the token's sequence, p = softmax(scale * qfull[t, h] . row_j)
    with row_j the cache row [r + rd] and c_j its first r values; float32 scores and sums."""
    _dev(out, qfull, cache, tables)
    T = qfull.shape[0]
    R = r + rd
    if tuple(qfull.shape) != (T, heads * R) or tuple(out.shape) != (T, heads * r) or out.dtype != qfull.dtype \
            or cache.dtype != qfull.dtype or tuple(cache.shape[1:]) != (PAGE, R) \
            or not (out.is_contiguous() and qfull.is_contiguous() and cache.is_contiguous()):
        raise KernelError("attn_latent: shapes do not agree")
    _check(_fn("attention_latent", "oe_attn_latent", out.dtype)(
        _ptr(out), _ptr(qfull), _ptr(cache), _ptr(tables), tables.shape[1], _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), T, heads, r,
        rd, float(scale), _stream()), "attn_latent")


def head_matmul(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[t, h, :] = w[h] @ a[t, h, :] for all heads in one launch: a [T, H, K] and out [T, H, N] views whose last axis
    is contiguous (token and head strides free), w [H, N, K] contiguous; a and w of one dtype, out of that dtype or float32."""
    _dev(out, a, w)
    T, H, K = a.shape
    N = w.shape[1]
    if tuple(w.shape) != (H, N, K) or tuple(out.shape) != (T, H, N) or a.stride(2) != 1 or out.stride(2) != 1 \
            or not w.is_contiguous() or a.dtype != w.dtype or out.dtype not in (a.dtype, torch.float32):
        raise KernelError("head_matmul: a [T, H, K], w [H, N, K] of one dtype, out [T, H, N] of that dtype or float32")
    fn = _fn("attention_latent", "oe_head_matmul", out.dtype) if out.dtype == a.dtype else \
        _fn("attention_latent", "oe_head_matmul", out.dtype, in_dtype=a.dtype)
    _check(fn(
        _ptr(out), out.stride(0), out.stride(1), _ptr(a), a.stride(0), a.stride(1), _ptr(w), T, H, N, K, _stream()),
        "head_matmul")


# ---------------------------------------------------------------------------------------- recurrent.cu

def short_conv_prepare(out_qkv, out_gb, proj, conv_w, conv_state, A_log, dt_bias, ctx, kv_heads: int, heads: int,
                       dk: int, dv: int, q_scale: float) -> None:
    """The inputs of a gated delta rule from the float32 projection rows [q | k | v | gate | beta | a]: see
    csrc/recurrent.cu.  conv_w [C, taps], conv_state [slots, max(taps - 1, 1), C], C = 2 G dk + H dv."""
    _dev(out_qkv, out_gb, proj, conv_w, conv_state, A_log, dt_bias)
    for t, n in ((out_qkv, "out_qkv"), (out_gb, "out_gb"), (proj, "proj"), (conv_w, "conv_w"),
                 (conv_state, "conv_state"), (A_log, "A_log"), (dt_bias, "dt_bias")):
        _f32c(t, n)
    T, P = proj.shape
    C = 2 * kv_heads * dk + heads * dv
    taps = conv_w.shape[1]
    if P != C + heads * dv + 2 * heads or tuple(conv_w.shape) != (C, taps) or tuple(out_qkv.shape) != (T, C) \
            or tuple(out_gb.shape) != (T, 2 * heads) or tuple(conv_state.shape[1:]) != (max(taps - 1, 1), C):
        raise KernelError("short_conv_prepare: shapes do not agree")
    _check(_fn("recurrent", "oe_short_conv_prepare")(
        _ptr(out_qkv), _ptr(out_gb), _ptr(proj), P, _ptr(conv_w), taps, _ptr(conv_state), _ptr(A_log), _ptr(dt_bias),
        _ptr(ctx.tok_seq), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), T, kv_heads, heads, dk, dv, float(q_scale), _stream()),
        "short_conv_prepare")


def conv_state_update(conv_state, proj, C: int, taps: int, ctx) -> None:
    """conv_state[slot] = the last taps - 1 rows (first C columns) that the sequence has brought so far."""
    _dev(conv_state, proj)
    _f32c(conv_state, "conv_state")
    _f32c(proj, "proj")
    if taps <= 1:
        return
    _check(_fn("recurrent", "oe_conv_state_update")(_ptr(conv_state), _ptr(proj), proj.shape[1], C, taps,
                                                    _ptr(ctx.seq_slot), _ptr(ctx.cu_q), ctx.n_seqs, _stream()),
           "conv_state_update")


def delta_rule_scan(o, state, qkv, gb, ctx, kv_heads: int, heads: int, dk: int, dv: int) -> None:
    """Per sequence and head, over the step's tokens in order: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  state [slots, H, dk, dv] float32 is read and written."""
    _dev(o, state, qkv, gb)
    for t, n in ((o, "o"), (state, "state"), (qkv, "qkv"), (gb, "gb")):
        _f32c(t, n)
    T = qkv.shape[0]
    if tuple(state.shape[1:]) != (heads, dk, dv) or tuple(o.shape) != (T, heads * dv) \
            or qkv.shape[1] != 2 * kv_heads * dk + heads * dv or tuple(gb.shape) != (T, 2 * heads):
        raise KernelError("delta_rule_scan: shapes do not agree")
    _check(_fn("recurrent", "oe_delta_rule_scan")(_ptr(o), _ptr(state), _ptr(qkv), _ptr(gb), _ptr(ctx.seq_slot),
                                                  _ptr(ctx.cu_q), ctx.n_seqs, kv_heads, heads, dk, dv, _stream()),
           "delta_rule_scan")


def token_shift_mix(out, h, mu, prev_state, ctx) -> None:
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]; the row before a step's first row is prev_state[slot]."""
    _dev(out, h, mu, prev_state)
    _f32c(mu, "mu")
    _f32c(prev_state, "prev_state")
    T, D = h.shape
    n_mix = mu.shape[0]
    if tuple(out.shape) != (n_mix, T, D) or out.dtype != h.dtype or not (out.is_contiguous() and h.is_contiguous()) \
            or mu.shape[1] != D or prev_state.shape[1] != D:
        raise KernelError("token_shift_mix: shapes do not agree")
    _check(_fn("recurrent", "oe_token_shift_mix", h.dtype)(
        _ptr(out), _ptr(h), _ptr(mu), _ptr(prev_state), n_mix, T, D, _ptr(ctx.tok_seq), _ptr(ctx.seq_slot),
        _ptr(ctx.cu_q), _stream()), "token_shift_mix")


def last_rows_to_state(state, h, ctx) -> None:
    """state[slot] = the sequence's last row of h in this step."""
    _dev(state, h)
    _f32c(state, "state")
    if not h.is_contiguous() or state.shape[1] != h.shape[1]:
        raise KernelError("last_rows_to_state: shapes do not agree")
    _check(_fn("recurrent", "oe_last_rows_to_state", h.dtype)(_ptr(state), _ptr(h), h.shape[1], _ptr(ctx.seq_slot),
                                                              _ptr(ctx.cu_q), ctx.n_seqs, _stream()),
           "last_rows_to_state")


def decay_scan(o, state, r, k, v, z, u, w0, ctx, heads: int, d: int) -> None:
    """Per sequence and head, over the step's tokens in order: o = (S + diag(u) k v^T)^T r;
    S <- diag(w) S + k v^T with w = exp(-exp(z + w0)).  r, k, v, z: float32 [T, H d] with one common row stride."""
    _dev(o, state, r, k, v, z, u, w0)
    for t, n in ((o, "o"), (state, "state"), (u, "u"), (w0, "w0")):
        _f32c(t, n)
    T = r.shape[0]
    stride = r.stride(0)
    for t in (r, k, v, z):
        if t.dtype != torch.float32 or t.stride(1) != 1 or t.stride(0) != stride or tuple(t.shape) != (T, heads * d):
            raise KernelError("decay_scan: r, k, v, z must be float32 [T, H d] with one row stride")
    if tuple(state.shape[1:]) != (heads, d, d) or tuple(o.shape) != (T, heads * d) or u.numel() != heads * d \
            or w0.numel() != heads * d:
        raise KernelError("decay_scan: shapes do not agree")
    _check(_fn("recurrent", "oe_decay_scan")(_ptr(o), _ptr(state), _ptr(r), _ptr(k), _ptr(v), _ptr(z), stride, _ptr(u),
                                             _ptr(w0), _ptr(ctx.seq_slot), _ptr(ctx.cu_q), ctx.n_seqs, heads, d,
                                             _stream()), "decay_scan")


_argmax_scratch: dict = {}


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of row r (float32 logits)."""
    _dev(logits, out)
    _i32(out, "out")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("argmax_rows: logits must be contiguous float32")
    rows, V = logits.shape
    if V >= 8192 and rows <= 4096:
        # wide vocabulary: slices of a row on different SMs, then one warp per row
        key = (logits.device.index, rows)
        sc = _argmax_scratch.get(key)
        if sc is None:
            sc = (torch.empty(rows * 32, dtype=torch.float32, device=logits.device),
                  torch.empty(rows * 32, dtype=torch.int32, device=logits.device))
            _argmax_scratch[key] = sc
        _check(_fn("sampling", "oe_argmax_rows_wide")(_ptr(logits), _ptr(out), _ptr(sc[0]), _ptr(sc[1]), rows, V,
                                                      _stream()), "argmax_rows")
        LAUNCHES[0] += 1
        return
    _check(_fn("sampling", "oe_argmax_rows")(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], _stream()),
           "argmax_rows")


def sample_rows(logits: torch.Tensor, out: torch.Tensor, row_slot: torch.Tensor, temperature: float, top_k: int,
                top_p: float, repeat_penalty: float, repeat_last_n: int, rng_seed: torch.Tensor,
                rng_counter: torch.Tensor, hist: torch.Tensor | None, hist_count: torch.Tensor | None,
                record: bool = True) -> None:
    """One token per row of float32 logits (overwritten), by the reference's sampling chain."""
    _dev(logits, out, row_slot, rng_seed, rng_counter, hist, hist_count)
    _i32(out, "out")
    _i32(row_slot, "row_slot")
    _i32(rng_counter, "rng_counter")
    if rng_seed.dtype != torch.int64:
        raise KernelError("sample_rows: rng_seed must be int64")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("sample_rows: logits must be contiguous float32")
    cap = 0
    if hist is not None:
        _i32(hist, "hist")
        _i32(hist_count, "hist_count")
        cap = hist.shape[1]
    _check(_fn("sampling", "oe_sample_rows")(
        _ptr(logits), _ptr(out), _ptr(row_slot), logits.shape[0], logits.shape[1], float(temperature), int(top_k),
        float(top_p), float(repeat_penalty), int(repeat_last_n), _ptr(rng_seed), _ptr(rng_counter), _ptr(hist),
        _ptr(hist_count), cap, int(record), _stream()), "sample_rows")
