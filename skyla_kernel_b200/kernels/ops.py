"""Python faces of the CUDA launchers: tensors in, one kernel launch each.

Every function checks device, dtype and layout, passes raw pointers and the
current CUDA stream to an ``extern "C"`` launcher, and raises
:class:`KernelError` with the launcher's message on a refused size or a failed
launch.  Nothing here computes on the host or falls back to library code.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors; there is no host path")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what}: expected a contiguous int32 tensor")
    return t


_FUNCS = {}


def _fn(module: str, name: str, argtypes):
    key = (module, name)
    f = _FUNCS.get(key)
    if f is None:
        lib = build.load(module)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _FUNCS[key] = f
    return f


#: kernel launches made through this module since import (bench.py reports the difference)
LAUNCHES = 0


def _check(module: str, rc: int):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        msg = build.load(module).skyla_error_message().decode("utf-8", "replace")
        raise KernelError(msg or f"{module}: error {rc}")


# ------------------------------------------------------------------ embedding
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[tokens[t], :]; tokens were checked against the vocabulary on the host."""
    _cuda(tokens, table, out)
    _i32(tokens, "tokens")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    n, hidden = tokens.numel(), table.shape[1]
    if out.shape[0] < n or out.shape[1] != hidden:
        raise KernelError(f"embed_gather: out {tuple(out.shape)} does not hold [{n}, {hidden}]")
    f = _fn("embed", "skyla_embed_gather",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int64, c_void_p])
    _check("embed", f(_ptr(tokens), n, _ptr(table), dtype_code(table), hidden, _ptr(out),
                      dtype_code(out), _rows(out, "out"), _stream()))
    return out


# ----------------------------------------------------------------------- norm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight, computed in 32-bit."""
    _cuda(x, weight, out, rows)
    _i32(rows, "rows")
    if weight.dtype != torch.float32 or not weight.is_contiguous():
        raise KernelError("rmsnorm: the weight must be a contiguous float32 vector")
    width = weight.numel()
    n = rows.numel() if rows is not None else x.shape[0]
    if x.shape[1] != width or out.shape[1] != width or out.shape[0] < n:
        raise KernelError(f"rmsnorm: shapes x {tuple(x.shape)} out {tuple(out.shape)} weight [{width}]")
    f = _fn("norm", "skyla_rmsnorm",
            [c_void_p, c_int, c_int64, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_int,
             c_int64, c_void_p])
    _check("norm", f(_ptr(x), dtype_code(x), _rows(x, "x"), _ptr(rows), n, width, _ptr(weight),
                     float(eps), _ptr(out), dtype_code(out), _rows(out, "out"), _stream()))
    return out


# --------------------------------------------------------------------- linear
STORE, ACCUMULATE, GATED = 0, 1, 2


def linear_plain(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, mode: int = STORE,
                 glu_group: int = 0) -> torch.Tensor:
    """y = x @ w.T (store), y += x @ w.T (accumulate, y float32) or the gated product.

    In gated mode ``w`` has ``2 * y.shape[1]`` rows in groups of ``glu_group``
    gate rows followed by the ``glu_group`` up rows of the same outputs.
    """
    _cuda(x, w, y)
    if not w.is_contiguous() or w.dim() != 2:
        raise KernelError("linear: the weight must be a contiguous matrix")
    m, k = x.shape
    n = y.shape[1]
    if w.shape[1] != k or w.shape[0] != (2 * n if mode == GATED else n) or y.shape[0] != m:
        raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} mode {mode}")
    f = _fn("linear_plain", "skyla_linear_plain",
            [c_void_p, c_int, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int64,
             c_int, c_int, c_void_p])
    _check("linear_plain", f(_ptr(x), dtype_code(x), _rows(x, "x"), _ptr(w), dtype_code(w), m, n, k,
                             _ptr(y), dtype_code(y), _rows(y, "y"), mode, glu_group or n, _stream()))
    return y


# ------------------------------------------------------------ attention parts
def qk_norm_rope_cache(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, nq: int, nkv: int,
                       hd: int, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                       eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                       n_rot: int, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                       k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       page_table: torch.Tensor, page_size: int) -> None:
    """Per-head norm and rotation of the new tokens; q in place, k and v into the cache.

    ``k_pool``/``v_pool`` of shape [pages, nkv, page_size, hd]; ``None`` skips the
    cache write (a run that reads another entry's cache).
    """
    _cuda(qkv, q_norm, k_norm, cos, sin, tok_pos, tok_slot, k_pool, v_pool, page_table)
    for t, what in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (page_table, "page_table")):
        _i32(t, what)
    for t, what in ((q_norm, "q_norm"), (k_norm, "k_norm"), (cos, "cos"), (sin, "sin")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{what}: expected a contiguous float32 tensor")
    n = tok_pos.numel()
    if k_pool is not None:
        if (k_pool.shape != v_pool.shape or tuple(k_pool.shape[1:]) != (nkv, page_size, hd)
                or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
            raise KernelError(f"cache pools {tuple(k_pool.shape)} do not match [pages, {nkv}, {page_size}, {hd}]")
        cdt = dtype_code(k_pool)
    else:
        cdt = dtype_code(qkv)
    if cos is not None and (cos.shape != sin.shape or cos.shape[1] != n_rot // 2):
        raise KernelError("rotary table does not match the rotary width")
    f = _fn("attn_prep", "skyla_qk_norm_rope_cache",
            [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_int, c_int, c_void_p])
    _check("attn_prep", f(_ptr(qkv), dtype_code(qkv), _rows(qkv, "qkv"), q_off, k_off, v_off, n, nq,
                          nkv, hd, _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos), _ptr(sin),
                          n_rot if cos is not None else 0, _ptr(tok_pos), _ptr(tok_slot),
                          _ptr(k_pool), _ptr(v_pool), cdt, _ptr(page_table), page_table.shape[1],
                          page_size, _stream()))


def attention_plain(q: torch.Tensor, out: torch.Tensor, nq: int, nkv: int, hd: int,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                    page_size: int, tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float,
                    window: int = 0) -> torch.Tensor:
    """Causal (optionally windowed) attention of each token over its own sequence's cache.

    ``q`` is [tokens, >= nq*hd] with contiguous rows (a view into a fused buffer
    is fine), ``out`` [tokens, nq*hd].
    """
    _cuda(q, out, k_pool, v_pool, page_table, tok_pos, tok_slot)
    for t, what in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (page_table, "page_table")):
        _i32(t, what)
    if q.dtype != out.dtype:
        raise KernelError("attention: q and out must share a dtype")
    if tuple(k_pool.shape[1:]) != (nkv, page_size, hd) or k_pool.shape != v_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not match [pages, {nkv}, {page_size}, {hd}]")
    n = tok_pos.numel()
    f = _fn("attention_plain", "skyla_attention_plain",
            [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p])
    _check("attention_plain", f(_ptr(q), dtype_code(q), _rows(q, "q"), _ptr(out), _rows(out, "out"), n,
                                nq, nkv, hd, _ptr(k_pool), _ptr(v_pool), dtype_code(k_pool),
                                _ptr(page_table), page_table.shape[1], page_size, _ptr(tok_pos),
                                _ptr(tok_slot), float(scale), int(window or 0), _stream()))
    return out


# ------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float = 0.0, top_k: int = 0,
           top_p: float = 1.0, seed: int = 0, req_ids: Optional[torch.Tensor] = None,
           steps: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits: argmax when ``temperature`` is 0, else a seeded draw."""
    _cuda(logits, out, req_ids, steps)
    _i32(out, "out"); _i32(req_ids, "req_ids"); _i32(steps, "steps")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    n, vocab = logits.shape
    if out.numel() < n:
        raise KernelError("sample: output too small")
    f = _fn("sampling", "skyla_sample",
            [c_void_p, c_int64, c_int, c_int, c_float, c_int, c_float, c_uint64, c_void_p, c_void_p,
             c_void_p, c_void_p])
    _check("sampling", f(_ptr(logits), _rows(logits, "logits"), n, vocab, float(temperature),
                         int(top_k), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_ids),
                         _ptr(steps), _ptr(out), _stream()))
    return out


# ------------------------------------------------------------------ utilities
def bandwidth_read(buf: torch.Tensor, blocks: int, sink: torch.Tensor) -> None:
    _cuda(buf, sink)
    f = _fn("util", "skyla_bandwidth_read", [c_void_p, c_size_t, c_int, c_void_p, c_void_p])
    _check("util", f(_ptr(buf), buf.numel() * buf.element_size(), blocks, _ptr(sink), _stream()))


def fill_normal(out: torch.Tensor, mean: float, std: float, seed: int) -> torch.Tensor:
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_normal: tensor must be contiguous")
    f = _fn("util", "skyla_fill_normal", [c_void_p, c_int, c_size_t, c_float, c_float, c_uint64, c_void_p])
    _check("util", f(_ptr(out), dtype_code(out), out.numel(), float(mean), float(std),
                     int(seed) & 0xFFFFFFFFFFFFFFFF, _stream()))
    return out
