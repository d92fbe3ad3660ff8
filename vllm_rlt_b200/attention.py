"""Paged verify attention on the B200 kernels, behind the reference's backend interface.

``B200PagedAttention`` is a kernel object with the call signature of the reference's
``TritonPagedAttention`` (``vllm_rlt/kernels/paged_attention.py:116-128``):

    kernel(q, key_cache, value_cache, block_tables, context_lengths) -> Tensor
    kernel.prefill(q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q, max_seqlen_q)

and ``create_backend`` wraps it as the reference's ``AttentionBackend(kernel, capabilities, info)``
(``vllm_rlt/attention/backend.py:15-57``) so it can be injected with
``KVCacheManager(..., attention=create_backend(device, dtype, head_dim, block_size))``.

Contract kept from the reference: the result is a new tensor shaped like ``q``; inputs are only
read; the K/V arguments are one layer's strided view of the pool and their strides are
honoured; everything is launched on the current stream with no host synchronisation and no host
read of the lengths (CUDA-graph capturable); an empty batch gives an empty result; a row of
length zero gives zeros and never dereferences its block table.  Misuse raises ``ValueError``
before any launch; kernel errors propagate — there is no fallback.
"""

from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Callable

import torch

from . import _capi


@dataclass(frozen=True)
class BackendCapabilities:
    """Same fields as the reference's ``BackendCapabilities`` (attention/backend.py:15-27)."""

    packed_prefill: bool = False
    cuda_graphs: bool = False
    async_scheduling: bool = False
    packed_matches_decode: bool = False
    device_context_lengths: bool = False
    sliding_window: bool = False


@dataclass
class AttentionBackend:
    """Same shape as the reference's ``AttentionBackend`` adapter (attention/backend.py:30-55)."""

    kernel: Callable
    capabilities: BackendCapabilities
    info: dict = field(default_factory=dict)

    def __call__(self, *args, **kwargs):
        return self.kernel(*args, **kwargs)

    def prefill(self, *args, **kwargs):
        return self.kernel.prefill(*args, **kwargs)

    def windowed(self, *args, **kwargs):
        method = getattr(self.kernel, "windowed", None)
        if method is None:
            selected = self.info.get("selected_backend", "this attention backend")
            raise NotImplementedError(f"{selected} does not implement sliding-window masking")
        return method(*args, **kwargs)

    @property
    def generation(self):
        return None


# Grouped (packed) rows are bit-identical to the same rows scored one at a time, so the
# speculative runner may verify with packed metadata (worker/speculative.py:176-178).
B200_CAPABILITIES = BackendCapabilities(
    packed_prefill=True,
    cuda_graphs=True,
    async_scheduling=True,
    packed_matches_decode=True,
    device_context_lengths=True,
    sliding_window=True,
)


class B200PagedAttention:
    """Depth-aware paged-KV attention for verification and decode rows."""

    def __init__(self):
        self._retired: list[torch.Tensor] = []      # outgrown scratch buffers (see _workspace)
        self._workspaces: dict[tuple[int, int], torch.Tensor] = {}
        self._planned: dict[tuple[int, int], tuple] = {}  # workspace key -> metadata the plan was built for
        self._sharing = 0

    @contextmanager
    def shared_plan(self):
        """Reuse the row grouping / work list across the layers of one depth pass.

        Inside this context, consecutive calls on one stream that pass the *same* block-table,
        length (and ``cu_seqlens_q``) tensors plan once and then only run, as the reference's
        model loop hands one metadata object to all 24 layers (``models/ouro.py:283-291``).
        "The same" means the same storage AND the same contents: a tensor that was rewritten in
        place since the plan was built (its version counter moved) is planned again, so a stale
        plan is never reused.  Tensors that carry no version counter (created under
        ``torch.inference_mode``) are planned on every call.  Outside the context every call
        plans for itself.
        """
        self._sharing += 1
        try:
            yield self
        finally:
            self._sharing -= 1
            if self._sharing == 0:
                self._planned.clear()

    def _workspace(self, device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
        # One scratch buffer per (device, stream): calls on one stream are ordered, calls on
        # different streams never share scratch.  Grown (doubling, by at most 256 MiB beyond the need),
        # never shrunk — and an outgrown buffer is kept, not freed: a caller's captured CUDA graph may have
        # this library's kernels baked in with that buffer as their scratch, and memory returned to the
        # allocator would be handed to someone else while the graph goes on replaying over it.
        key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
        buffer = self._workspaces.get(key)
        if buffer is None or buffer.numel() < nbytes:
            if buffer is not None:
                self._retired.append(buffer)
            size = max(nbytes, 0 if buffer is None else min(2 * buffer.numel(), nbytes + (256 << 20)))
            buffer = torch.empty(size, dtype=torch.uint8, device=device)
            self._workspaces[key] = buffer
            self._planned.pop(key, None)
        return buffer

    @staticmethod
    def _versions(*tensors):
        """In-place modification counters of the metadata tensors, or None if one has none."""
        try:
            return tuple(-1 if t is None else t._version for t in tensors)
        except RuntimeError:
            return None

    @staticmethod
    def _check_cache(q, key_cache, value_cache):
        if q.dim() != 3:
            raise ValueError("q must be [rows, heads, head_dim]")
        if key_cache.dim() != 4 or value_cache.shape != key_cache.shape:
            raise ValueError("key_cache/value_cache must be [blocks, block_size, kv_heads, head_dim]")
        if key_cache.stride() != value_cache.stride():
            raise ValueError("key_cache and value_cache must share one layout")
        if q.dtype not in _capi.DTYPE_CODES or key_cache.dtype != q.dtype or value_cache.dtype != q.dtype:
            raise ValueError("q, key_cache and value_cache must share a float32/float16/bfloat16 dtype")
        if key_cache.shape[3] != q.shape[2]:
            raise ValueError("head_dim of q and the KV cache differ")
        if q.shape[1] % key_cache.shape[2] != 0:
            raise ValueError("query heads must be a positive multiple of KV heads")
        if key_cache.stride(3) != 1 or key_cache.stride(2) != key_cache.shape[3]:
            raise ValueError("the [kv_heads, head_dim] tail of the KV cache view must be contiguous")

    def _run(self, q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q):
        device = _capi.require_cuda(q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q)
        self._check_cache(q, key_cache, value_cache)
        if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
            raise ValueError("block tables must be contiguous int32 [rows, pages]")
        if context_lengths.dtype != torch.int32 or context_lengths.dim() != 1:
            raise ValueError("context_lengths must be int32 [rows]")
        q = q.contiguous()
        rows = q.shape[0]
        out = torch.empty_like(q)
        if rows == 0:
            return out
        table_rows, width = block_tables.shape
        if cu_seqlens_q is None:
            if table_rows != rows or context_lengths.numel() != rows:
                raise ValueError("one block-table row and one context length per query row")
        else:
            if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_q.numel() != table_rows + 1:
                raise ValueError("cu_seqlens_q must be int32 [sequences + 1]")
            if context_lengths.numel() != table_rows:
                raise ValueError("one context length per packed sequence")
            cu_seqlens_q = cu_seqlens_q.contiguous()
        context_lengths = context_lengths.contiguous()
        lib = _capi.load()
        blocks, block_size, kv_heads, head_dim = key_cache.shape
        with torch.cuda.device(device):
            stream = _capi.stream_of(q)
            nbytes = lib.rlt_verify_attention_workspace_bytes(rows, q.shape[1], kv_heads, head_dim,
                                                              block_size, max(width, 1))
            ws_key = (device.index if device.index is not None else torch.cuda.current_device(), stream.value or 0)
            workspace = self._workspace(device, stream.value or 0, nbytes)
            dtype = _capi.DTYPE_CODES[q.dtype]
            call_args = (
                _capi.ptr(q), _capi.ptr(out), _capi.ptr(key_cache), _capi.ptr(value_cache),
                key_cache.stride(0), key_cache.stride(1), blocks, block_size, q.shape[1], kv_heads,
                head_dim, dtype, _capi.ptr(block_tables), table_rows, width,
                _capi.ptr(context_lengths), _capi.ptr(cu_seqlens_q), rows, _capi.ptr(workspace),
                workspace.numel(), stream)
            status = _capi.ERR_UNSUPPORTED
            versions = self._versions(block_tables, context_lengths, cu_seqlens_q) if self._sharing else None
            if versions is not None:
                plan_key = (block_tables.data_ptr(), table_rows, width, context_lengths.data_ptr(),
                            0 if cu_seqlens_q is None else cu_seqlens_q.data_ptr(), rows, q.shape[1], kv_heads,
                            head_dim, block_size, dtype, versions)
                if self._planned.get(ws_key) != plan_key:
                    status = lib.rlt_verify_attention_plan(
                        _capi.ptr(block_tables), table_rows, width, _capi.ptr(context_lengths),
                        _capi.ptr(cu_seqlens_q), rows, q.shape[1], kv_heads, head_dim, block_size, dtype,
                        _capi.ptr(workspace), workspace.numel(), stream)
                    if status == _capi.OK:
                        self._planned[ws_key] = plan_key
                if self._planned.get(ws_key) == plan_key:
                    status = lib.rlt_verify_attention_run(*call_args)
            if status == _capi.ERR_UNSUPPORTED:  # no shared plan, or a shape outside the tiled kernel
                self._planned.pop(ws_key, None)
                status = lib.rlt_verify_attention(*call_args)
        _capi.check(status, "verify_attention")
        return out

    def last_status(self, device=None) -> dict:
        """Diagnostics of the last tiled call on the current stream (synchronises the stream):
        work items planned, rows of length zero, the device-side error bits (0 = no wait gave up) and
        the claim counter (0 after a clean run)."""
        import ctypes

        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            workspace = self._workspaces.get((torch.cuda.current_device(), stream or 0))
            if workspace is None:
                raise RuntimeError("no tiled attention call has run on this stream")
            words = (ctypes.c_uint32 * 4)()
            status = _capi.load().rlt_verify_attention_status(_capi.ptr(workspace), ctypes.c_void_p(stream), words)
        _capi.check(status, "verify_attention_status")
        return {"items": words[0], "zero_rows": words[1], "error": words[2], "claim_counter": words[3]}

    def __call__(self, q, key_cache, value_cache, block_tables, context_lengths):
        return self._run(q, key_cache, value_cache, block_tables, context_lengths, None)

    def windowed(self, q, key_cache, value_cache, block_tables, context_lengths, window):
        """Row r attends only its last ``window`` keys, its own position included; keys outside the
        window stay stored (``torch_paged_attention_windowed``, kernels/paged_attention.py:39-70 of the
        reference, reached through ``KVCacheManager._attend_windowed``, core/kv_cache_manager.py:773-803).
        One block-table row per query row; ``ValueError`` for a window that is not a positive ``int``."""
        if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
            raise ValueError("window must be a positive integer")
        device = _capi.require_cuda(q, key_cache, value_cache, block_tables, context_lengths)
        self._check_cache(q, key_cache, value_cache)
        if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
            raise ValueError("block tables must be contiguous int32 [rows, pages]")
        rows = q.shape[0]
        if context_lengths.dtype != torch.int32 or context_lengths.shape != (rows,) or block_tables.shape[0] != rows:
            raise ValueError("one block-table row and one int32 context length per query row")
        q = q.contiguous()
        out = torch.empty_like(q)
        if rows == 0:
            return out
        blocks, block_size, kv_heads, head_dim = key_cache.shape
        with torch.cuda.device(device):
            status = _capi.load().rlt_windowed_attention(
                _capi.ptr(q), _capi.ptr(out), _capi.ptr(key_cache), _capi.ptr(value_cache), key_cache.stride(0),
                key_cache.stride(1), blocks, block_size, q.shape[1], kv_heads, head_dim, _capi.DTYPE_CODES[q.dtype],
                _capi.ptr(block_tables), block_tables.shape[1], _capi.ptr(context_lengths.contiguous()), rows,
                min(window, 2**31 - 1), _capi.stream_of(q))
        _capi.check(status, "windowed_attention")
        return out

    def prefill(self, q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q, max_seqlen_q):
        """Packed rows: one block-table row per sequence, bottom-right causal lengths.

        Sequences of at most 16 new tokens (verification rows in packed form) go through the
        grouped verify kernel and are bit-identical to the same rows scored one at a time
        (`packed_matches_decode`); longer ones (prompts) through the prefill kernel, 64 query
        tokens per CTA, which agrees with it to the dtype's tolerance.
        """
        if int(max_seqlen_q) <= 16:
            return self._run(q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q)
        device = _capi.require_cuda(q, key_cache, value_cache, block_tables, context_lengths, cu_seqlens_q)
        self._check_cache(q, key_cache, value_cache)
        if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or not block_tables.is_contiguous():
            raise ValueError("block tables must be contiguous int32 [sequences, pages]")
        sequences, width = block_tables.shape
        if context_lengths.dtype != torch.int32 or context_lengths.shape != (sequences,):
            raise ValueError("context_lengths must be int32 [sequences]")
        if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_q.shape != (sequences + 1,):
            raise ValueError("cu_seqlens_q must be int32 [sequences + 1]")
        q = q.contiguous()
        out = torch.empty_like(q)
        rows = q.shape[0]
        if rows == 0 or sequences == 0:
            return out
        lib = _capi.load()
        blocks, block_size, kv_heads, head_dim = key_cache.shape
        with torch.cuda.device(device):
            stream = _capi.stream_of(q)
            nbytes = lib.rlt_prefill_attention_workspace_bytes(rows, sequences, q.shape[1], kv_heads, head_dim,
                                                               block_size, max(width, 1))
            lengths, cu = context_lengths.contiguous(), cu_seqlens_q.contiguous()
            for attempt in range(2):
                workspace = self._workspace(device, stream.value or 0, nbytes)
                status = lib.rlt_prefill_attention(
                    _capi.ptr(q), _capi.ptr(out), _capi.ptr(key_cache), _capi.ptr(value_cache), key_cache.stride(0),
                    key_cache.stride(1), blocks, block_size, q.shape[1], kv_heads, head_dim, _capi.DTYPE_CODES[q.dtype],
                    _capi.ptr(block_tables), sequences, width, _capi.ptr(lengths), _capi.ptr(cu), rows,
                    _capi.ptr(workspace), workspace.numel(), stream)
                if status != _capi.ERR_WORKSPACE or attempt == 1:
                    break
                # the rows fall back to the grouped kernel (32-bit dtype, or caches the tensor map cannot express)
                nbytes = lib.rlt_verify_attention_workspace_bytes(rows, q.shape[1], kv_heads, head_dim, block_size, max(width, 1))
        _capi.check(status, "prefill_attention")
        return out


def create_backend(device, dtype: torch.dtype, head_dim: int, block_size: int) -> AttentionBackend:
    """The B200 backend as an ``AttentionBackend``; explicit selection, no fallback.

    Mirrors ``_create_explicit`` of the reference (attention/backend.py:80-99): validates the
    hardware and configuration and raises ``ValueError`` when they do not fit.
    """
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("the B200 attention backend requires a CUDA device")
    if dtype not in _capi.DTYPE_CODES:
        raise ValueError("KV dtype must be float32, float16, or bfloat16")
    if head_dim > 256:
        raise ValueError("the B200 attention backend supports head_dim <= 256")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    if torch.cuda.get_device_capability(device)[0] != 10:
        raise ValueError("the B200 attention backend is built for sm_100a only")
    _capi.load()
    info = {
        "backend": "b200",
        "requested_backend": "b200",
        "selected_backend": "b200",
        "selection_reason": "explicitly requested b200",
        "tiled_kernel": bool(dtype != torch.float32 and head_dim == 128 and block_size == 16),
    }
    return AttentionBackend(B200PagedAttention(), B200_CAPABILITIES, info)
