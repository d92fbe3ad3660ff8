"""Fused elementwise pieces of a decoder layer around the attention call.

Host-side mirror of `apply_rotary_pos_emb` + `KVCacheManager._write_prepared` as
`OuroAttention.forward` chains them (`vllm_rlt/models/ouro.py:179-186` of the reference) and of
`RMSNorm.forward` with the sandwich residual adds of `OuroDecoderLayer.forward`
(`vllm_rlt/layers/normalization.py:20-23`, `models/ouro.py:217-221`).
"""

from __future__ import annotations

import torch

from . import _capi


def _heads_view(t: torch.Tensor, name: str):
    if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
        raise ValueError(f"{name} must be [rows, heads, head_dim] with a contiguous [heads, head_dim] tail")


def rope_kv_write(q, k, v, cos, sin, key_cache, value_cache, write_blocks, write_offsets, write_mask=None,
                  active_rows=None):
    """Rotate q and k, write the rotated k and v into their pages, return the rotated q.

    `q`, `k`, `v` may be slices of one fused projection output (any row stride).  `cos`, `sin`:
    `[rows, head_dim]` (or `[rows, 1, head_dim]`) in the model dtype, as `RotaryEmbedding.forward`
    returns them.  `key_cache` / `value_cache` are one layer's `[blocks, block, kv_heads,
    head_dim]` views; the addressing arguments are those of `kv_write`.  The result is bit-identical
    to `q * cos + rotate_half(q) * sin` (and the same for k) on tensors of that dtype.
    """
    _capi.require_cuda(q, k, v, cos, sin, key_cache, value_cache, write_blocks, write_offsets, write_mask,
                       active_rows)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _heads_view(t, name)
    rows, q_heads, head_dim = q.shape
    kv_heads = k.shape[1]
    if k.shape != (rows, kv_heads, head_dim) or v.shape != k.shape or head_dim % 2:
        raise ValueError("k and v must be [rows, kv_heads, head_dim] with an even head_dim")
    if not (q.dtype == k.dtype == v.dtype == key_cache.dtype == value_cache.dtype) or q.dtype not in _capi.DTYPE_CODES:
        raise ValueError("q, k, v and the cache must share one of float32 / float16 / bfloat16")
    cos, sin = cos.reshape(rows, head_dim), sin.reshape(rows, head_dim)
    if cos.dtype != q.dtype or sin.dtype != q.dtype:
        raise ValueError("cos and sin must have the model dtype")
    if key_cache.dim() != 4 or key_cache.shape[2:] != (kv_heads, head_dim) or key_cache.stride(3) != 1 \
            or key_cache.stride(2) != head_dim or key_cache.stride() != value_cache.stride() \
            or key_cache.shape != value_cache.shape:
        raise ValueError("cache views must be [blocks, block, kv_heads, head_dim] with equal strides")
    for name, t in (("write_blocks", write_blocks), ("write_offsets", write_offsets)):
        if t.dtype != torch.int64 or t.shape != (rows,):
            raise ValueError(f"{name} must be int64 [rows]")
    mask = None
    if write_mask is not None:
        if write_mask.shape != (rows,) or write_mask.dtype not in (torch.bool, torch.uint8):
            raise ValueError("write_mask must be bool [rows]")
        mask = write_mask.contiguous().view(torch.uint8)
    if active_rows is not None and (active_rows.dtype != torch.int32 or active_rows.numel() != 1):
        raise ValueError("active_rows must be a 0-dim int32 tensor")
    q_out = torch.empty((rows, q_heads, head_dim), dtype=q.dtype, device=q.device)
    if rows == 0:
        return q_out
    cos, sin = cos.contiguous(), sin.contiguous()
    write_blocks, write_offsets = write_blocks.contiguous(), write_offsets.contiguous()
    with torch.cuda.device(q.device):
        code = _capi.load().rlt_rope_kv_write(
            _capi.ptr(q), q.stride(0), _capi.ptr(k), k.stride(0), _capi.ptr(v), v.stride(0),
            _capi.ptr(cos), _capi.ptr(sin), _capi.ptr(q_out), _capi.ptr(key_cache),
            _capi.ptr(value_cache), key_cache.stride(0), key_cache.stride(1), key_cache.shape[0], key_cache.shape[1],
            q_heads, kv_heads, head_dim, _capi.DTYPE_CODES[q.dtype], _capi.ptr(write_blocks),
            _capi.ptr(write_offsets), _capi.ptr(mask), _capi.ptr(active_rows), rows, _capi.stream_of(q))
    _capi.check(code, "rope_kv_write")
    return q_out


def sandwich_norm(x, weight, eps: float, residual=None, weight2=None, *, in_place: bool = False):
    """`total = [residual +] weight * rmsnorm(x)` and, with `weight2`, `norm = weight2 * rmsnorm(total)`.

    Returns `(total, norm)` (`norm` is None without `weight2`).  `in_place` writes `total` over
    `residual` (the residual stream of a decoder layer).  Roundings are those of the tensor
    expressions in the model dtype; the mean of squares is accumulated in double.
    """
    _capi.require_cuda(x, weight, residual, weight2)
    if x.dim() != 2 or not x.is_contiguous() or x.dtype not in _capi.DTYPE_CODES:
        raise ValueError("x must be contiguous [rows, hidden] float32 / float16 / bfloat16")
    rows, hidden = x.shape
    for name, w in (("weight", weight), ("weight2", weight2)):
        if w is not None and (w.shape != (hidden,) or w.dtype != x.dtype or not w.is_contiguous()):
            raise ValueError(f"{name} must be contiguous [hidden] of x's dtype")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise ValueError("residual must match x")
    if in_place and residual is None:
        raise ValueError("in_place needs a residual")
    total = residual if in_place else torch.empty_like(x)
    norm = None if weight2 is None else torch.empty_like(x)
    if rows == 0:
        return total, norm
    with torch.cuda.device(x.device):
        code = _capi.load().rlt_sandwich_norm(_capi.ptr(x), _capi.ptr(weight), _capi.ptr(residual), _capi.ptr(total),
                                              _capi.ptr(weight2), _capi.ptr(norm), rows, hidden, float(eps),
                                              _capi.DTYPE_CODES[x.dtype], _capi.stream_of(x))
    _capi.check(code, "sandwich_norm")
    return total, norm
