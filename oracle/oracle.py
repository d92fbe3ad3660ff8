"""ctypes front end of the CPU oracle (``oracle/rlt_oracle.c``).

TEST INFRASTRUCTURE ONLY.  The oracle is the checker for the CUDA kernels and the
timed CPU baseline of ``bench.py``; only ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline legs may import this module.  The product package
(``vllm_rlt_b200``) never does, and fails loudly when its CUDA library is missing.

Every function takes CPU ``torch`` tensors (bf16 has no numpy type) and mirrors the
argument order of the C-ABI entry point it checks (``include/rlt_verify.h``).
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_ref" / "librlt_oracle.so"
_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_lib = None


def build(force: bool = False) -> Path:
    """Compile the oracle with the recipe in ``oracle/Makefile``."""
    if force or not _LIB_PATH.exists():
        subprocess.run(["make", "-C", str(_HERE)] + (["-B"] if force else []), check=True,
                       capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.orc_probabilities.restype = ctypes.c_int
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def _p(t):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.device.type == "cpu"
    return ctypes.c_void_p(t.data_ptr())


def _i64(x):
    return ctypes.c_int64(int(x))


def _cache_geometry(cache):
    """[num_blocks, block_size, kv_heads, head_dim] view -> (block_stride, token_stride)."""
    assert cache.dim() == 4 and cache.stride(3) == 1 and cache.stride(2) == cache.shape[3]
    return cache.stride(0), cache.stride(1)


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(gate)
    lib().orc_silu_and_mul(_p(gate), _p(up), _p(out), _i64(gate.numel()), _DTYPES[gate.dtype])
    return out


def kv_write(key_cache, value_cache, k, v, write_blocks, write_offsets, write_mask=None,
             active_rows=None):
    bs, ts = _cache_geometry(key_cache)
    assert _cache_geometry(value_cache) == (bs, ts)
    k, v = k.contiguous(), v.contiguous()
    mask = None if write_mask is None else write_mask.to(torch.uint8).contiguous()
    lib().orc_kv_write(_p(key_cache), _p(value_cache), _i64(bs), _i64(ts), key_cache.shape[2],
                       key_cache.shape[3], _DTYPES[key_cache.dtype], _p(k), _p(v),
                       _p(write_blocks.contiguous()), _p(write_offsets.contiguous()), _p(mask),
                       _p(active_rows), k.shape[0])


def paged_attention(q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q=None):
    bs, ts = _cache_geometry(key_cache)
    assert _cache_geometry(value_cache) == (bs, ts)
    q = q.contiguous()
    out = torch.empty_like(q)
    tables = block_tables.to(torch.int32).contiguous()
    lens = context_lengths.to(torch.int32).contiguous()
    cu = None if cu_seqlens_q is None else cu_seqlens_q.to(torch.int32).contiguous()
    lib().orc_paged_attention(_p(q), _p(out), _p(key_cache), _p(value_cache), _i64(bs), _i64(ts),
                              key_cache.shape[1], q.shape[1], key_cache.shape[2], q.shape[2],
                              _DTYPES[q.dtype], _p(tables), tables.shape[0],
                              tables.shape[1] if tables.dim() == 2 else 0, _p(lens), _p(cu),
                              q.shape[0])
    return out


def paged_attention_windowed(q, key_cache, value_cache, block_tables, context_lengths, window):
    bs, ts = _cache_geometry(key_cache)
    assert _cache_geometry(value_cache) == (bs, ts) and type(window) is int and window > 0
    q = q.contiguous()
    out = torch.empty_like(q)
    tables = block_tables.to(torch.int32).contiguous()
    lens = context_lengths.to(torch.int32).contiguous()
    lib().orc_paged_attention_windowed(_p(q), _p(out), _p(key_cache), _p(value_cache), _i64(bs), _i64(ts),
                                       key_cache.shape[1], q.shape[1], key_cache.shape[2], q.shape[2],
                                       _DTYPES[q.dtype], _p(tables), tables.shape[1], _p(lens), q.shape[0], window)
    return out


def argmax_rows(logits):
    assert logits.dim() == 2 and logits.stride(1) == 1
    targets = torch.empty(logits.shape[0], dtype=torch.int64)
    lib().orc_argmax_rows(_p(logits), _i64(logits.stride(0)), logits.shape[0], logits.shape[1],
                          _DTYPES[logits.dtype], _p(targets))
    return targets


def accept_greedy(logits, cu_rows, tokens, starts, slots=None, slot_values=None, row_counts=None):
    rows, n = logits.shape[0], cu_rows.numel() - 1
    result = torch.empty(rows + 2 * n, dtype=torch.int64)
    lib().orc_accept_greedy(_p(logits), _i64(logits.stride(0)), rows, logits.shape[1],
                            _DTYPES[logits.dtype], _p(cu_rows), n, _p(row_counts), _p(tokens), tokens.shape[1],
                            _p(starts), _p(slots), _p(slot_values), _p(result))
    return result


def probabilities(logits_row, temperature, top_k=-1, top_p=1.0):
    probs = torch.empty(logits_row.numel(), dtype=torch.float32)
    status = lib().orc_probabilities(_p(logits_row.contiguous()), logits_row.numel(),
                                     _DTYPES[logits_row.dtype], ctypes.c_float(temperature),
                                     int(top_k), ctypes.c_float(top_p), _p(probs))
    return probs, status


def sample_rows(logits, temperature, uniforms, top_k=None, top_p=None):
    rows = logits.shape[0]
    tokens = torch.empty(rows, dtype=torch.int64)
    status = torch.empty(rows, dtype=torch.int32)
    lib().orc_sample_rows(_p(logits), _i64(logits.stride(0)), rows, logits.shape[1],
                          _DTYPES[logits.dtype], _p(temperature), _p(top_k), _p(top_p), _p(uniforms),
                          _p(tokens), _p(status))
    return tokens, status


def accept_rejection(target_logits, draft_logits, cu_rows, tokens, starts, temperature, u_accept,
                     u_final, slots=None, slot_values=None, top_k=None, top_p=None, row_counts=None):
    rows, n = target_logits.shape[0], cu_rows.numel() - 1
    assert target_logits.stride() == draft_logits.stride()
    result = torch.empty(rows + 2 * n, dtype=torch.int64)
    status = torch.empty(n, dtype=torch.int32)
    lib().orc_accept_rejection(_p(target_logits), _p(draft_logits), _i64(target_logits.stride(0)),
                               rows, target_logits.shape[1], _DTYPES[target_logits.dtype],
                               _p(cu_rows), n, _p(row_counts), _p(tokens), tokens.shape[1], _p(starts),
                               _p(temperature), _p(top_k), _p(top_p), _p(u_accept), _p(u_final), _p(slots),
                               _p(slot_values), _p(result), _p(status))
    return result, status


def round_uniforms(seeds, rounds, width):
    """(u_draft [n, width], u_accept [n, width], u_final [n]) of a round, float32."""
    n = seeds.numel()
    u_draft, u_accept = torch.empty(n, width), torch.empty(n, width)
    u_final = torch.empty(n)
    lib().orc_round_uniforms(_p(seeds.contiguous()), _p(rounds.contiguous()), n, width, _p(u_draft), _p(u_accept),
                             _p(u_final))
    return u_draft, u_accept, u_final


def philox4x32_10(counter, key):
    """One Philox4x32-10 block (four 32-bit words) for a 4-word counter and a 2-word key."""
    c = (ctypes.c_uint32 * 4)(*counter)
    k = (ctypes.c_uint32 * 2)(*key)
    out = (ctypes.c_uint32 * 4)()
    lib().orc_philox4x32_10(c, k, out)
    return list(out)


def finalize_tokens(key_pool, value_pool, tables, slots, depths, positions):
    assert key_pool.dim() == 5 and key_pool.stride() == value_pool.stride()
    lib().orc_finalize_tokens(_p(key_pool), _p(value_pool), _i64(key_pool.stride(0)), _i64(key_pool.stride(1)),
                              _i64(key_pool.stride(2)), key_pool.shape[1], key_pool.shape[2], key_pool.shape[3],
                              key_pool.shape[4], _DTYPES[key_pool.dtype], _p(tables.contiguous()), tables.shape[1],
                              tables.shape[2], _p(slots.contiguous()), _p(depths.contiguous()),
                              _p(positions.contiguous()), slots.numel())


def pipeline_shift(state, widths, row_starts, choices, step_hidden, limits, draft_loops, target_loops):
    """In place on `state` (dict of tokens, depths, candidates, active(uint8), hidden, token, position); returns result."""
    n, width = state["tokens"].shape
    result = torch.zeros(6 * n, dtype=torch.int64)
    lib().orc_pipeline_shift(_p(state["tokens"]), _p(state["depths"]), _p(state["candidates"]), _p(state["active"]),
                             _p(state["hidden"]), _p(state["token"]), _p(state["position"]), _p(widths),
                             _p(row_starts), _p(choices), _p(step_hidden.contiguous()), _p(limits), n, width,
                             state["hidden"].shape[2], _DTYPES[state["hidden"].dtype], draft_loops, target_loops,
                             _p(result))
    return result


def rollback(starts, emitted, tables, block_size, pages_used=None, refcounts=None,
             written_prefix=None):
    n, planes, width = tables.shape
    layers = 0 if written_prefix is None else written_prefix.shape[2]
    frontier = torch.zeros(n, dtype=torch.int64)
    context_lengths = torch.zeros(n, dtype=torch.int32)
    write_blocks = torch.zeros(n, planes, dtype=torch.int64)
    write_offsets = torch.zeros(n, dtype=torch.int64)
    status = torch.zeros(n, dtype=torch.int32)
    lib().orc_rollback(_p(starts), _p(emitted), n, _p(tables.contiguous()), planes, width,
                       block_size, _p(pages_used), _p(refcounts),
                       _i64(0 if refcounts is None else refcounts.numel()), _p(written_prefix),
                       layers, _p(frontier), _p(context_lengths), _p(write_blocks),
                       _p(write_offsets), _p(status))
    return frontier, context_lengths, write_blocks, write_offsets, status


def rope_kv_write(q, k, v, cos, sin, key_cache, value_cache, write_blocks, write_offsets, write_mask=None,
                  active_rows=None):
    """q, k, v: [rows, heads, head_dim] views with contiguous [heads, head_dim] tails; returns rotated q."""
    bs, ts = _cache_geometry(key_cache)
    assert _cache_geometry(value_cache) == (bs, ts)
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == t.shape[2]
    q_out = torch.empty(q.shape, dtype=q.dtype)
    mask = None if write_mask is None else write_mask.to(torch.uint8).contiguous()
    lib().orc_rope_kv_write(_p(q), _i64(q.stride(0)), _p(k), _i64(k.stride(0)), _p(v), _i64(v.stride(0)),
                            _p(cos.contiguous()), _p(sin.contiguous()), _p(q_out), _p(key_cache), _p(value_cache),
                            _i64(bs), _i64(ts), q.shape[1], k.shape[1], q.shape[2], _DTYPES[q.dtype],
                            _p(write_blocks.contiguous()), _p(write_offsets.contiguous()), _p(mask),
                            _p(active_rows), q.shape[0])
    return q_out


def sandwich_norm(x, weight, eps, residual=None, weight2=None):
    """Returns (sum, norm): sum = [residual +] weight * T(rmsnorm(x)); norm = weight2 * T(rmsnorm(sum)) or None."""
    x = x.contiguous()
    total = torch.empty_like(x)
    norm = None if weight2 is None else torch.empty_like(x)
    lib().orc_sandwich_norm(_p(x), _p(weight.contiguous()), _p(None if residual is None else residual.contiguous()),
                            _p(total), _p(None if weight2 is None else weight2.contiguous()), _p(norm), x.shape[0],
                            x.shape[1], ctypes.c_float(eps), _DTYPES[x.dtype])
    return total, norm
