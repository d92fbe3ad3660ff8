"""KV-cache side of the verify step: writing new K/V rows and rolling back rejected positions.

``kv_write`` mirrors the tensor contract of ``KVCacheManager._write_prepared``
(``vllm_rlt/core/kv_cache_manager.py:675-701``) and of the graph variant
``_DeviceCache._write_prepared`` (``vllm_rlt/worker/cuda_graph.py:108-120``).
``rollback`` is the device form of ``KVCacheManager.truncate_suffix`` (:338-356) plus the slot
mapping the next round derives from the new frontier (``worker/async_speculative.py:272-281``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _capi


def kv_write(key_cache, value_cache, k, v, write_blocks, write_offsets, write_mask=None,
             active_rows=None) -> None:
    """``cache[write_blocks, write_offsets] = k`` (and v) for the active rows of one layer view.

    key_cache / value_cache: one layer's view ``[blocks, block_size, kv_heads, head_dim]``.
    write_blocks / write_offsets: int64 ``[rows]``.  write_mask: bool ``[rows]`` or None.
    active_rows: 0-dim int32 device tensor or None.  Inactive rows load no address.
    """
    _capi.require_cuda(key_cache, value_cache, k, v, write_blocks, write_offsets, write_mask, active_rows)
    if key_cache.dim() != 4 or value_cache.shape != key_cache.shape or key_cache.stride() != value_cache.stride():
        raise ValueError("key_cache/value_cache must be matching [blocks, block_size, kv_heads, head_dim] views")
    if key_cache.stride(3) != 1 or key_cache.stride(2) != key_cache.shape[3]:
        raise ValueError("the [kv_heads, head_dim] tail of the KV cache view must be contiguous")
    rows = k.shape[0]
    expected = (rows, key_cache.shape[2], key_cache.shape[3])
    if tuple(k.shape) != expected or tuple(v.shape) != expected:
        raise ValueError("k and v must be [rows, kv_heads, head_dim]")
    if k.dtype != key_cache.dtype or v.dtype != key_cache.dtype or key_cache.dtype not in _capi.DTYPE_CODES:
        raise ValueError("KV dtype must be float32, float16, or bfloat16 and match the cache")
    for name, t in (("write_blocks", write_blocks), ("write_offsets", write_offsets)):
        if t.dtype != torch.int64 or t.shape != (rows,):
            raise ValueError(f"{name} must have shape [rows] and use torch.int64")
    if write_mask is not None and (write_mask.dtype != torch.bool or write_mask.shape != (rows,)):
        raise ValueError("write_mask must be bool [rows] on the cache device")
    if active_rows is not None and (active_rows.dtype != torch.int32 or active_rows.numel() != 1):
        raise ValueError("active_rows must be a 0-dim int32 device tensor")
    if rows == 0:
        return
    k, v = k.contiguous(), v.contiguous()
    write_blocks, write_offsets = write_blocks.contiguous(), write_offsets.contiguous()
    write_mask = None if write_mask is None else write_mask.contiguous()
    with torch.cuda.device(key_cache.device):
        status = _capi.load().rlt_kv_write(
            _capi.ptr(key_cache), _capi.ptr(value_cache), key_cache.stride(0), key_cache.stride(1),
            key_cache.shape[0], key_cache.shape[1], key_cache.shape[2], key_cache.shape[3],
            _capi.DTYPE_CODES[key_cache.dtype], _capi.ptr(k), _capi.ptr(v),
            _capi.ptr(write_blocks), _capi.ptr(write_offsets),
            _capi.ptr(write_mask),
            _capi.ptr(active_rows), rows, _capi.stream_of(key_cache))
    _capi.check(status, "kv_write")


def finalize_tokens(key_pool, value_pool, tables, slots, depths, positions) -> None:
    """Copy each token's exit-depth K/V (all layers) into every deeper plane of its request.

    The batched device form of `KVCacheManager.finalize_token` (core/kv_cache_manager.py:805-831).
    key_pool / value_pool: the whole pool `[blocks, layers, block_size, kv_heads, head_dim]`;
    tables: int32 `[slots, planes, pages]`; slots / depths / positions: int64 `[rows]`.
    """
    _capi.require_cuda(key_pool, value_pool, tables, slots, depths, positions)
    if key_pool.dim() != 5 or value_pool.shape != key_pool.shape or key_pool.stride() != value_pool.stride():
        raise ValueError("key_pool/value_pool must be matching [blocks, layers, block_size, kv_heads, head_dim] pools")
    if key_pool.stride(4) != 1 or key_pool.stride(3) != key_pool.shape[4]:
        raise ValueError("the [kv_heads, head_dim] tail of the KV pool must be contiguous")
    if key_pool.dtype not in _capi.DTYPE_CODES or value_pool.dtype != key_pool.dtype:
        raise ValueError("KV dtype must be float32, float16, or bfloat16")
    if tables.dim() != 3 or tables.dtype != torch.int32:
        raise ValueError("tables must be int32 [slots, planes, pages]")
    rows = slots.numel()
    for name, t in (("slots", slots), ("depths", depths), ("positions", positions)):
        if t.dtype != torch.int64 or t.shape != (rows,):
            raise ValueError(f"{name} must be int64 [rows]")
    if rows == 0:
        return
    blocks, layers, block_size, kv_heads, head_dim = key_pool.shape
    tables, slots, depths, positions = tables.contiguous(), slots.contiguous(), depths.contiguous(), positions.contiguous()
    with torch.cuda.device(key_pool.device):
        status = _capi.load().rlt_finalize_tokens(
            _capi.ptr(key_pool), _capi.ptr(value_pool), key_pool.stride(0), key_pool.stride(1), key_pool.stride(2),
            blocks, layers, block_size, kv_heads, head_dim, _capi.DTYPE_CODES[key_pool.dtype],
            _capi.ptr(tables), tables.shape[1], tables.shape[2], _capi.ptr(slots),
            _capi.ptr(depths), _capi.ptr(positions), rows, _capi.stream_of(key_pool))
    _capi.check(status, "finalize_tokens")


@dataclass
class RollbackResult:
    """Device tensors describing the state after rollback (one entry per request)."""

    frontier: torch.Tensor          # int64 [n]  start + emitted
    context_lengths: torch.Tensor   # int32 [n]  frontier + 1: keys visible to the next input token
    write_blocks: torch.Tensor      # int64 [n, planes]  page of the next input token, per plane
    write_offsets: torch.Tensor     # int64 [n]
    status: torch.Tensor            # int32 [n]  0 ok, 4 shared page refused, 5 position outside table


def rollback(starts, emitted, tables, block_size, *, pages_used=None, refcounts=None,
             written_prefix=None) -> RollbackResult:
    """Roll every request back to ``starts + emitted`` on the device.

    tables: int32 ``[n, planes, pages]`` (never modified).  written_prefix: int64
    ``[n, planes, layers]`` validity frontiers, clamped in place.  refcounts: int32 ``[blocks]``;
    a request whose pages at or after the frontier page are shared is refused (status 4) and
    left untouched, as ``truncate_suffix`` raises ``ValueError`` for it.
    """
    device = _capi.require_cuda(starts, emitted, tables, pages_used, refcounts, written_prefix)
    if tables.dim() != 3 or tables.dtype != torch.int32:
        raise ValueError("tables must be int32 [requests, planes, pages]")
    n, planes, width = tables.shape
    for name, t in (("starts", starts), ("emitted", emitted)):
        if t.dtype != torch.int64 or t.shape != (n,):
            raise ValueError(f"{name} must be int64 [requests]")
    layers = 0
    if written_prefix is not None:
        if written_prefix.dtype != torch.int64 or written_prefix.dim() != 3 or not written_prefix.is_contiguous():
            raise ValueError("written_prefix must be contiguous int64 [requests, planes, layers]")
        layers = written_prefix.shape[2]
    result = RollbackResult(
        frontier=torch.empty(n, dtype=torch.int64, device=device),
        context_lengths=torch.zeros(n, dtype=torch.int32, device=device),
        write_blocks=torch.zeros(n, planes, dtype=torch.int64, device=device),
        write_offsets=torch.zeros(n, dtype=torch.int64, device=device),
        status=torch.zeros(n, dtype=torch.int32, device=device),
    )
    if n == 0:
        return result
    starts, emitted, tables = starts.contiguous(), emitted.contiguous(), tables.contiguous()
    with torch.cuda.device(device):
        status = _capi.load().rlt_rollback(
            _capi.ptr(starts), _capi.ptr(emitted), n,
            _capi.ptr(tables), planes, width, block_size, _capi.ptr(pages_used),
            _capi.ptr(refcounts), 0 if refcounts is None else refcounts.numel(),
            _capi.ptr(written_prefix), layers, _capi.ptr(result.frontier),
            _capi.ptr(result.context_lengths), _capi.ptr(result.write_blocks),
            _capi.ptr(result.write_offsets), _capi.ptr(result.status), _capi.stream_of(tables))
    _capi.check(status, "rollback")
    return result
