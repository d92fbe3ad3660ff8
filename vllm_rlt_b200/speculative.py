"""Acceptance side of the verify step: argmax, greedy acceptance, draws, rejection sampling.

Host-side mirror of ``greedy_accept`` / ``rejection_sample`` (``vllm_rlt/worker/speculative.py:32-63``),
of the device acceptance ``AsyncSpeculativeRunner._accept_and_update_state``
(``vllm_rlt/worker/async_speculative.py:417-447``) and of ``Sampler.sample``
(``vllm_rlt/worker/sampler.py:62-81``), batched over requests and with explicit uniforms
in place of a ``torch.Generator``.

Verification rows are request-major: request ``i`` owns rows ``cu_rows[i] .. cu_rows[i+1]-1``.
``tokens[i, 0]`` is the committed input token, ``tokens[i, 1:c_i]`` its drafts.  The result
buffer has the reference's wire layout (async_speculative.py:62-77):
``[per-row tokens (rows) | accepted (n) | next_position (n)]``, int64.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _capi


@dataclass
class SpeculativeResult:
    """Same fields as ``vllm_rlt/worker/output.py:20-25``."""

    token_ids: list
    accepted_count: int
    kv_frontier: int | None = None


def _check_logits(logits):
    if logits.dim() != 2 or logits.stride(1) != 1 or logits.dtype not in _capi.DTYPE_CODES:
        raise ValueError("logits must be [rows, vocab] float32/float16/bfloat16 with unit inner stride")


def _check_round(rows, cu_rows, tokens, starts, slots, slot_values, row_counts=None, result=None):
    n = cu_rows.numel() - 1
    if cu_rows.dtype != torch.int32 or cu_rows.dim() != 1 or n < 0:
        raise ValueError("cu_rows must be int32 [requests + 1]")
    if row_counts is not None and (row_counts.dtype != torch.int32 or row_counts.shape != (n,)):
        raise ValueError("row_counts must be int32 [requests]")
    if result is not None and (result.dtype != torch.int64 or result.dim() != 1 or result.numel() < rows + 2 * n
                               or not result.is_contiguous()):
        raise ValueError("result must be contiguous int64 with at least rows + 2 * requests elements")
    if tokens.dtype != torch.int64 or tokens.dim() != 2 or tokens.shape[0] != n or not tokens.is_contiguous():
        raise ValueError("tokens must be contiguous int64 [requests, width]")
    if starts.dtype != torch.int64 or starts.shape != (n,):
        raise ValueError("starts must be int64 [requests]")
    if (slots is None) != (slot_values is None):
        raise ValueError("slots and slot_values go together")
    if slots is not None:
        if slots.dtype != torch.int64 or slots.shape != (n,):
            raise ValueError("slots must be int64 [requests]")
        if slot_values.dtype != torch.int64 or slot_values.dim() != 2 or slot_values.shape[1] != 2 \
                or not slot_values.is_contiguous():
            raise ValueError("slot_values must be contiguous int64 [slots, 2]")
    return n


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """``logits.argmax(-1)`` (lowest index on ties) as int64 on the device."""
    _capi.require_cuda(logits)
    _check_logits(logits)
    targets = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    if logits.shape[0] == 0:
        return targets
    with torch.cuda.device(logits.device):
        status = _capi.load().rlt_argmax_rows(_capi.ptr(logits), logits.stride(0), logits.shape[0],
                                              logits.shape[1], _capi.DTYPE_CODES[logits.dtype],
                                              _capi.ptr(targets), _capi.stream_of(logits))
    _capi.check(status, "argmax_rows")
    return targets


def accept_greedy(logits, cu_rows, tokens, starts, slots=None, slot_values=None, result=None, row_counts=None):
    """Greedy acceptance of a whole round on the device; returns the int64 wire buffer.

    ``result[:rows]`` are the target ids of every verification row, ``result[rows:rows+n]``
    the accepted counts, ``result[rows+n:]`` the next positions; ``slot_values[slots[i]]``
    receives ``(next_token, next_position)``.  No generator is touched.  ``row_counts`` (int32
    ``[n]``) marks how many rows of each request's span are real in a round of fixed shape; the
    padding rows get -1 and a request without rows is left alone.
    """
    _capi.require_cuda(logits, cu_rows, tokens, starts, slots, slot_values, result, row_counts)
    _check_logits(logits)
    rows = logits.shape[0]
    n = _check_round(rows, cu_rows, tokens, starts, slots, slot_values, row_counts, result)
    if result is None:
        result = torch.empty(rows + 2 * n, dtype=torch.int64, device=logits.device)
    if n == 0:
        return result
    # contiguous copies are bound to names so that they outlive the launch
    cu_rows, starts = cu_rows.contiguous(), starts.contiguous()
    row_counts = None if row_counts is None else row_counts.contiguous()
    slots = None if slots is None else slots.contiguous()
    with torch.cuda.device(logits.device):
        status = _capi.load().rlt_accept_greedy(
            _capi.ptr(logits), logits.stride(0), rows, logits.shape[1], _capi.DTYPE_CODES[logits.dtype],
            _capi.ptr(cu_rows), n, _capi.ptr(row_counts), _capi.ptr(tokens), tokens.shape[1], _capi.ptr(starts),
            _capi.ptr(slots), _capi.ptr(slot_values), _capi.ptr(result), _capi.stream_of(logits))
    _capi.check(status, "accept_greedy")
    return result


def _check_filters(top_k, top_p, count, what):
    """top_k int32 [count] (<= 0 or >= vocab: off) and top_p float32 [count] (>= 1: off), or None."""
    if top_k is not None and (top_k.dtype != torch.int32 or top_k.shape != (count,)):
        raise ValueError(f"top_k must be int32 [{what}]")
    if top_p is not None and (top_p.dtype != torch.float32 or top_p.shape != (count,)):
        raise ValueError(f"top_p must be float32 [{what}]")
    return (None if top_k is None else top_k.contiguous()), (None if top_p is None else top_p.contiguous())


def probabilities(logits, temperature, top_k=None, top_p=None):
    """``Sampler.probabilities`` (``vllm_rlt/worker/sampler.py:27-55``) for every row at once.

    ``softmax(float(logits) / temperature)`` over the strict top-k support (ties to the lower
    index), trimmed to the top-p nucleus, renormalised.  Returns ``(probs float32 [rows, vocab],
    status int32 [rows])``.  ``temperature`` must be positive: greedy decoding has no
    temperature-scaled distribution (such rows get status 3 and zeros; the reference raises
    ``ValueError``).
    """
    _capi.require_cuda(logits, temperature, top_k, top_p)
    _check_logits(logits)
    rows, vocab = logits.shape
    if temperature.dtype != torch.float32 or temperature.shape != (rows,):
        raise ValueError("temperature must be float32 [rows]")
    top_k, top_p = _check_filters(top_k, top_p, rows, "rows")
    probs = torch.empty(rows, vocab, dtype=torch.float32, device=logits.device)
    status = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    if rows == 0:
        return probs, status
    temperature = temperature.contiguous()      # bound to a name: it must outlive the launch
    with torch.cuda.device(logits.device):
        code = _capi.load().rlt_probabilities(
            _capi.ptr(logits), logits.stride(0), rows, vocab, _capi.DTYPE_CODES[logits.dtype],
            _capi.ptr(temperature), _capi.ptr(top_k), _capi.ptr(top_p), _capi.ptr(probs),
            _capi.ptr(status), _capi.stream_of(logits))
    _capi.check(code, "probabilities")
    return probs, status


def sample_rows(logits, temperature, uniforms, top_k=None, top_p=None):
    """One draw per row from the row's sampling distribution (see ``probabilities``);
    temperature 0 is argmax.

    Returns ``(tokens int64 [rows], status int32 [rows])``.
    """
    _capi.require_cuda(logits, temperature, uniforms, top_k, top_p)
    _check_logits(logits)
    rows = logits.shape[0]
    for name, t in (("temperature", temperature), ("uniforms", uniforms)):
        if t.dtype != torch.float32 or t.shape != (rows,):
            raise ValueError(f"{name} must be float32 [rows]")
    top_k, top_p = _check_filters(top_k, top_p, rows, "rows")
    tokens = torch.empty(rows, dtype=torch.int64, device=logits.device)
    status = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    if rows == 0:
        return tokens, status
    temperature, uniforms = temperature.contiguous(), uniforms.contiguous()
    with torch.cuda.device(logits.device):
        code = _capi.load().rlt_sample_rows(
            _capi.ptr(logits), logits.stride(0), rows, logits.shape[1], _capi.DTYPE_CODES[logits.dtype],
            _capi.ptr(temperature), _capi.ptr(top_k), _capi.ptr(top_p),
            _capi.ptr(uniforms), _capi.ptr(tokens), _capi.ptr(status), _capi.stream_of(logits))
    _capi.check(code, "sample_rows")
    return tokens, status


def accept_rejection(target_logits, draft_logits, cu_rows, tokens, starts, temperature, u_accept, u_final,
                     slots=None, slot_values=None, result=None, top_k=None, top_p=None, row_counts=None,
                     status=None, workspace=None):
    """Rejection-sampling acceptance of a whole round; returns ``(result, status)``.

    ``result[cu_rows[i] : cu_rows[i] + accepted_i + 1]`` are request i's emitted tokens (its
    other rows hold -1); ``status[i]`` is 0, or 1 (zero proposal probability: ``ValueError`` in
    the reference), 2 (invalid residual mass: ``RuntimeError``), 3 (NaN / +inf logits).
    Use ``raise_for_status`` to turn them into those exceptions after the one host read of a
    round.  ``temperature[i] == 0`` takes the greedy branch for that request.  ``top_k`` /
    ``top_p`` are per request and filter both the target and the proposal distribution, as the
    reference builds both with the request's ``SamplingParams``.  ``row_counts`` as in
    ``accept_greedy``.  ``status`` (int32 ``[n]``) and ``workspace`` (uint8, at least
    ``rlt_accept_rejection_workspace_bytes(rows)``) may be passed by a caller that owns its buffers.
    """
    _capi.require_cuda(target_logits, draft_logits, cu_rows, tokens, starts, temperature, u_accept, u_final,
                       slots, slot_values, result, top_k, top_p, row_counts, status, workspace)
    _check_logits(target_logits)
    _check_logits(draft_logits)
    if target_logits.shape != draft_logits.shape or target_logits.stride() != draft_logits.stride() \
            or target_logits.dtype != draft_logits.dtype:
        raise ValueError("target and draft logits must share shape, strides and dtype")
    rows = target_logits.shape[0]
    n = _check_round(rows, cu_rows, tokens, starts, slots, slot_values, row_counts, result)
    for name, t, count in (("temperature", temperature, n), ("u_accept", u_accept, rows), ("u_final", u_final, n)):
        if t.dtype != torch.float32 or t.shape != (count,):
            raise ValueError(f"{name} must be float32 [{count}]")
    top_k, top_p = _check_filters(top_k, top_p, n, "requests")
    if result is None:
        result = torch.empty(rows + 2 * n, dtype=torch.int64, device=target_logits.device)
    if status is None:
        status = torch.zeros(n, dtype=torch.int32, device=target_logits.device)
    elif status.dtype != torch.int32 or status.shape != (n,) or not status.is_contiguous():
        raise ValueError("status must be contiguous int32 [requests]")
    if n == 0:
        return result, status
    lib = _capi.load()
    need = lib.rlt_accept_rejection_workspace_bytes(rows)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=target_logits.device)
    elif workspace.dtype != torch.uint8 or workspace.numel() < need or not workspace.is_contiguous():
        raise ValueError(f"workspace must be contiguous uint8 with at least {need} bytes")
    cu_rows, starts, temperature = cu_rows.contiguous(), starts.contiguous(), temperature.contiguous()
    u_accept, u_final = u_accept.contiguous(), u_final.contiguous()
    row_counts = None if row_counts is None else row_counts.contiguous()
    slots = None if slots is None else slots.contiguous()
    with torch.cuda.device(target_logits.device):
        code = lib.rlt_accept_rejection(
            _capi.ptr(target_logits), _capi.ptr(draft_logits), target_logits.stride(0), rows,
            target_logits.shape[1], _capi.DTYPE_CODES[target_logits.dtype], _capi.ptr(cu_rows), n,
            _capi.ptr(row_counts), _capi.ptr(tokens), tokens.shape[1], _capi.ptr(starts), _capi.ptr(temperature),
            _capi.ptr(top_k), _capi.ptr(top_p), _capi.ptr(u_accept), _capi.ptr(u_final), _capi.ptr(slots),
            _capi.ptr(slot_values), _capi.ptr(result), _capi.ptr(status), _capi.ptr(workspace), workspace.numel(),
            _capi.stream_of(target_logits))
    _capi.check(code, "accept_rejection")
    return result, status


def round_uniforms(seeds, rounds, width: int):
    """Uniforms of one round: ``(u_draft [n, width], u_accept [n, width], u_final [n])``, float32.

    The device counterpart of the per-request generators of the reference's ``RngRegistry``
    (``vllm_rlt/worker/sampler.py:84-119``): a counter-based generator keyed by the request's
    seed and its round number, so no host generator has to be consulted between rounds and a
    request's draws do not depend on the batch it runs in.  ``seeds``, ``rounds``: int64 ``[n]``.
    """
    device = _capi.require_cuda(seeds, rounds)
    n = seeds.numel()
    for name, t in (("seeds", seeds), ("rounds", rounds)):
        if t.dtype != torch.int64 or t.shape != (n,):
            raise ValueError(f"{name} must be int64 [requests]")
    if not 1 <= width <= 4096:
        raise ValueError("width must be in [1, 4096]")
    u_draft = torch.empty(n, width, dtype=torch.float32, device=device)
    u_accept = torch.empty(n, width, dtype=torch.float32, device=device)
    u_final = torch.empty(n, dtype=torch.float32, device=device)
    if n == 0:
        return u_draft, u_accept, u_final
    seeds, rounds = seeds.contiguous(), rounds.contiguous()
    with torch.cuda.device(device):
        code = _capi.load().rlt_round_uniforms(_capi.ptr(seeds), _capi.ptr(rounds), n, width, _capi.ptr(u_draft),
                                               _capi.ptr(u_accept), _capi.ptr(u_final), _capi.stream_of(seeds))
    _capi.check(code, "round_uniforms")
    return u_draft, u_accept, u_final


@dataclass
class PipelineState:
    """Batched form of the reference's DevicePipelineState + per-request (token, position)
    (worker/async_speculative.py:28-50): `width` oldest-first slots per request, all on the device."""

    tokens: torch.Tensor       # int64 [n, width]
    depths: torch.Tensor       # int64 [n, width]
    candidates: torch.Tensor   # int64 [n, width]
    active: torch.Tensor       # bool  [n, width]
    hidden: torch.Tensor       # model dtype [n, width, hidden_size]
    token: torch.Tensor        # int64 [n]  last committed token
    position: torch.Tensor     # int64 [n]  its position


def pipeline_shift(state: PipelineState, widths, row_starts, choices, step_hidden, limits, *, draft_loops: int,
                   target_loops: int, result=None):
    """Apply one pipeline step's outcome to every request's device state, in place.

    The fused form of the per-request program at the end of `AsyncSpeculativeRunner._pipeline_step`
    (async_speculative.py:527-580): emit the head slot that reached `target_loops`, accept or reject its
    draft candidate, shift the surviving slots and their retained hidden rows, start the next draft slot
    (or restart from the corrected token), honour the output limit.  Returns the int64 wire buffer
    `[n, 6]` = prediction, accepted, emitted, next position, drafted count, verified count.
    """
    _capi.require_cuda(state.tokens, state.depths, state.candidates, state.active, state.hidden, state.token,
                       state.position, widths, row_starts, choices, step_hidden, limits, result)
    n, width = state.tokens.shape
    for name, t in (("tokens", state.tokens), ("depths", state.depths), ("candidates", state.candidates)):
        if t.dtype != torch.int64 or t.shape != (n, width) or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous int64 [requests, width]")
    if state.active.dtype != torch.bool or state.active.shape != (n, width) or not state.active.is_contiguous():
        raise ValueError("active must be contiguous bool [requests, width]")
    if state.hidden.dim() != 3 or state.hidden.shape[:2] != (n, width) or not state.hidden.is_contiguous() \
            or state.hidden.dtype not in _capi.DTYPE_CODES:
        raise ValueError("hidden must be contiguous [requests, width, hidden_size]")
    for name, t in (("token", state.token), ("position", state.position), ("limits", limits)):
        if t.dtype != torch.int64 or t.shape != (n,) or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous int64 [requests]")
    for name, t in (("widths", widths), ("row_starts", row_starts)):
        if t.dtype != torch.int32 or t.shape != (n,):
            raise ValueError(f"{name} must be int32 [requests]")
    if choices.dtype != torch.int64 or step_hidden.dtype != state.hidden.dtype \
            or step_hidden.shape != (choices.numel(), state.hidden.shape[2]):
        raise ValueError("choices must be int64 [rows] and step_hidden [rows, hidden_size] of the state dtype")
    if result is None:
        result = torch.empty(6 * n, dtype=torch.int64, device=state.tokens.device)
    if n == 0:
        return result.view(0, 6)
    widths, row_starts = widths.contiguous(), row_starts.contiguous()
    choices, step_hidden = choices.contiguous(), step_hidden.contiguous()
    with torch.cuda.device(state.tokens.device):
        status = _capi.load().rlt_pipeline_shift(
            _capi.ptr(state.tokens), _capi.ptr(state.depths), _capi.ptr(state.candidates), _capi.ptr(state.active),
            _capi.ptr(state.hidden), _capi.ptr(state.token), _capi.ptr(state.position),
            _capi.ptr(widths), _capi.ptr(row_starts), _capi.ptr(choices),
            _capi.ptr(step_hidden), _capi.ptr(limits), n, width, state.hidden.shape[2],
            _capi.DTYPE_CODES[state.hidden.dtype], draft_loops, target_loops, _capi.ptr(result),
            _capi.stream_of(state.tokens))
    _capi.check(status, "pipeline_shift")
    return result[: 6 * n].view(n, 6)


def raise_for_status(status_values) -> None:
    """Raise what the reference raises for a per-request status list already on the host."""
    for i, code in enumerate(status_values):
        if code == _capi.ROW_ZERO_PROPOSAL:
            raise ValueError(f"request {i}: candidate has zero proposal probability")
        if code == _capi.ROW_INVALID_RESIDUAL:
            raise RuntimeError(f"request {i}: invalid speculative residual probability mass")
        if code == _capi.ROW_BAD_LOGITS:
            raise RuntimeError(f"request {i}: non-finite logits in speculative acceptance")
        if code == _capi.ROW_SHARED_PAGE:
            raise ValueError(f"request {i}: cannot truncate shared prefix pages")
        if code == _capi.ROW_BAD_POSITION:
            raise ValueError(f"request {i}: invalid KV truncation frontier")


def decode_result(result_host, cu_rows_host) -> tuple[list[SpeculativeResult], list[int]]:
    """Split a round's wire buffer (already copied to the host) into per-request results.

    The decoding ``SpeculativeRoundTicket.collect`` performs (async_speculative.py:122-136):
    returns ``(results, frontiers)``.
    """
    n = len(cu_rows_host) - 1
    rows = cu_rows_host[-1]
    results = []
    for i in range(n):
        accepted = result_host[rows + i]
        start = cu_rows_host[i]
        results.append(SpeculativeResult(list(result_host[start : start + accepted + 1]), accepted))
    return results, list(result_host[rows + n : rows + 2 * n])
