"""The speculative runner of the verify step: submitted rounds with device-owned token state.

`B200SpeculativeRunner` has the runner-facing surface of the reference's `SpeculativeRunner` /
`AsyncSpeculativeRunner` (`vllm_rlt/worker/speculative.py:143-295`,
`vllm_rlt/worker/async_speculative.py:153-500`):

    ticket = runner.submit(batch)        # batch.requests: spans (request, token_start, token_count)
    ticket.ready()                       # has the round's result reached the host?
    output = ticket.collect()            # ModelRunnerOutput(speculative=[SpeculativeResult...], frontiers=[...])
    runner.release(request)              # a finished or cancelled request gives its slot back
    runner.stats                         # SpeculativeStats
    runner.snapshot_pipeline / restore_pipeline

and keeps the rules of the device-resident runner: a submission never reads the device
(`tests/test_async_speculative.py:151-158` of the reference patches `Tensor.item/tolist` to
raise while it submits two rounds), each request's `(input token, position)` lives in a device
slot table that one round's acceptance writes and the next round's draft reads, the host's
`token_start` is only a reservation bound, and at most two rounds are in flight.

What is different from the reference is the shape of a round.  The reference plans compact
row sets on the host for every draft offset and uploads their index tensors
(`_round_plan`, `async_speculative.py:329-368`).  Here a round has a FIXED shape for a given
number of requests `nb`: every draft pass has `nb` rows and the verify passes `nb * (K + 1)`
rows; rows a request does not use (its `token_count` is below `K + 1`, or it is padding of the
batch-size bucket) have context length 0 and a false write mask, so attention gives them no
work and nothing is written for them.  Everything between the slot table and the result
buffer — draft passes, LM head, proposals, verify passes, acceptance, slot update, rollback —
is therefore one static launch sequence, captured once per bucket as ONE CUDA graph, and a
submission is: one small pinned upload (slots, counts, round numbers), one graph launch, one
small download.  Sampled requests are supported in the same round (the reference's
device-resident runner is greedy only, `engine/stage_engine.py:327-332`): their uniforms come
from a counter-based generator keyed by the request's seed and round number
(`round_uniforms`), so no host generator is consulted.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _capi
from .kv_cache import rollback
from .speculative import (PipelineState, SpeculativeResult, accept_greedy, accept_rejection, argmax_rows,
                          pipeline_shift, raise_for_status, round_uniforms, sample_rows)


# ---- interface types (the fields of the reference's objects that the runner reads) ----------
@dataclass(frozen=True)
class SamplingParams:
    """vllm_rlt/sampling_params.py:6-17 of the reference (the fields that reach the runner)."""

    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = -1
    seed: int = 0

    def __post_init__(self):
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be a positive integer")
        if not self.temperature >= 0 or self.temperature == float("inf"):
            raise ValueError("temperature must be finite and nonnegative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k != -1 and self.top_k < 1:
            raise ValueError("top_k must be -1 or positive")
        if not 0 <= self.seed < 2 ** 63:
            raise ValueError("seed must be an integer in [0, 2**63)")


@dataclass
class Request:
    """vllm_rlt/request.py:37-108 of the reference, reduced to what speculation touches."""

    request_id: str
    prompt_token_ids: list
    sampling_params: SamplingParams
    generated_token_ids: list = field(default_factory=list)
    num_output_placeholders: int = 0
    num_speculative_rounds: int = 0
    finished: bool = False

    @property
    def num_scheduled_outputs(self) -> int:
        return len(self.generated_token_ids) + self.num_output_placeholders

    @property
    def position(self) -> int:
        return len(self.prompt_token_ids) + self.num_scheduled_outputs - 1

    @property
    def input_token_id(self) -> int:
        return self.generated_token_ids[-1]


@dataclass(frozen=True)
class ScheduledRequest:
    """A speculative span (vllm_rlt/core/scheduler.py:24-38)."""

    request: object
    token_start: int = 0
    token_count: int = 1


@dataclass(frozen=True)
class SchedulerOutput:
    """vllm_rlt/core/scheduler.py:41-48."""

    phase: object
    requests: list


@dataclass(frozen=True)
class SpeculativeConfig:
    """vllm_rlt/config.py:176-192 of the reference."""

    num_speculative_tokens: int
    draft_loops: int = 2
    target_loops: int = 4
    mode: str = "block"

    def __post_init__(self):
        for name in ("num_speculative_tokens", "draft_loops", "target_loops"):
            if type(getattr(self, name)) is not int or getattr(self, name) < 1:
                raise ValueError(f"{name} must be a positive integer")
        if self.mode not in ("block", "pipeline"):
            raise ValueError("speculative mode must be block or pipeline")
        if self.mode == "pipeline" and self.target_loops % self.draft_loops:
            raise ValueError("pipeline draft_loops must divide target_loops")
        if self.draft_loops >= self.target_loops:
            raise ValueError("draft_loops must be smaller than target_loops")


@dataclass
class SpeculativeStats:
    """vllm_rlt/worker/speculative.py:23-29."""

    rounds: int = 0
    drafted_tokens: int = 0
    accepted_tokens: int = 0
    committed_tokens: int = 0
    verified_rows: int = 0


@dataclass(frozen=True)
class ModelRunnerOutput:
    """The speculative fields of vllm_rlt/worker/output.py:27-36."""

    speculative: list | None = None
    frontiers: list | None = None
    completion: object = None


@dataclass
class SpeculativeRequestState:
    """vllm_rlt/worker/async_speculative.py:42-52: what the runner keeps per live request."""

    request: object
    slot: int
    submitted: int = 0
    delivered: int = 0
    event: object = None       # completion of the last round submitted for the request


class KVCacheManagerView:
    """The runner's view of a `vllm_rlt.core.kv_cache_manager.KVCacheManager` (or anything shaped like it):
    the LAST_EXITED pools as they are (`key_cache` / `value_cache`, `[blocks, layers, block, kv_heads,
    head_dim]`, core/kv_cache_manager.py:143-145) and a request's block tables, one per depth plane, from its
    allocation (`_get_allocation(request_id).block_tables`, :54-59).  `max_pages` bounds the pages of one
    request on one plane (its `max_tokens / block_size`).  The manager keeps allocating, growing and freeing;
    call `runner.refresh_tables(request)` after it has grown a request's tables."""

    def __init__(self, manager, max_pages: int):
        self.manager = manager
        self.key, self.value = manager.key_cache, manager.value_cache
        self.block, self.max_pages = manager.block_size, max_pages
        self.refcounts = None            # the manager refuses shared pages itself when the scheduler truncates

    def device_tables(self, request_id) -> torch.Tensor:
        tables = self.manager._get_allocation(request_id).block_tables
        width = max(len(t) for t in tables)
        if width > self.max_pages:
            raise ValueError("the request's block tables are wider than max_pages")
        host = torch.zeros(len(tables), width, dtype=torch.int32)
        for plane, table in enumerate(tables):
            host[plane, : len(table)] = torch.tensor(table, dtype=torch.int32)
        self._staging = host.pin_memory()                      # kept until the next call's copy is queued behind it
        return self._staging.to(self.key.device, non_blocking=True)


class _HostBuffer:
    """Pinned staging of one in-flight round (the reference's SpeculativeRoundBuffer,
    async_speculative.py:55-82): the plan that goes up and the wire record that comes down."""

    def __init__(self, plan_elements: int, wire_elements: int):
        self.plan = torch.empty(plan_elements, dtype=torch.int64, pin_memory=True)
        self.wire = torch.empty(wire_elements, dtype=torch.int64, pin_memory=True)
        self.leased = False
        self.done: torch.cuda.Event | None = None


class SpeculativeRoundTicket:
    """What `submit` returns (async_speculative.py:84-151)."""

    def __init__(self, runner, batch, buffer, states, nb, width, mode):
        self.runner, self.batch, self.buffer, self.states = runner, batch, buffer, states
        self.nb, self.width, self.mode = nb, width, mode
        self.rounds = tuple(s.submitted - 1 for s in states)
        self.cached: ModelRunnerOutput | None = None
        self.retired = False
        self.keepalive: list = []          # pinned staging of this submission's uploads

    @property
    def has_result(self):
        return True

    def ready(self) -> bool:
        return self.buffer.done.query()

    def collect(self) -> ModelRunnerOutput:
        """Wait for the round's record and decode it; raises what the reference raises for a
        request whose acceptance or rollback failed (`raise_for_status`)."""
        if self.cached is not None:
            return self.cached
        if self.retired:
            raise RuntimeError("cannot collect a retired speculative ticket")
        self.buffer.done.synchronize()
        n, nb, w = len(self.batch.requests), self.nb, self.width
        if self.mode == "pipeline":
            values = self.buffer.wire[: 6 * n].view(n, 6).tolist()
            self.cached = ModelRunnerOutput(
                speculative=[SpeculativeResult([token] if emitted else [], accepted)
                             for token, accepted, emitted, _, _, _ in values],
                frontiers=[row[3] for row in values])
            self.runner.stats.drafted_tokens += sum(row[4] for row in values)
            self.runner.stats.verified_rows += sum(row[5] for row in values)
        else:
            values = self.buffer.wire[: nb * w + 4 * nb].tolist()
            rows = nb * w
            try:
                raise_for_status(values[rows + 2 * nb: rows + 2 * nb + n])
                raise_for_status(values[rows + 3 * nb: rows + 3 * nb + n])
            except Exception:
                self.retire(discard=True)
                raise
            results = []
            for i in range(n):
                accepted = values[rows + i]
                results.append(SpeculativeResult(values[i * w: i * w + accepted + 1], accepted))
            frontiers = values[rows + nb: rows + nb + n]
            self.cached = ModelRunnerOutput(speculative=results,
                                            frontiers=frontiers if self.runner.report_frontiers else None)
        # Delivery is counted by whoever drives the runner in the device-resident protocol (the reference's
        # engine checks `state.delivered == round` and increments it, engine/stage_engine.py:738-752); in the
        # synchronous protocol nobody else would.  The staging buffer is free either way: its record is decoded.
        if not self.runner.report_frontiers:
            for state in self.states:
                state.delivered += 1
        self.retire()
        return self.cached

    def retire(self, *, discard: bool = False):
        """Give the round's staging buffer back (at most two rounds hold one at a time)."""
        if self.retired:
            return
        if self.cached is None:
            if not discard:
                raise RuntimeError("collect a speculative ticket before retiring its buffer")
            self.buffer.done.synchronize()
        self.buffer.leased = False
        self.retired = True


class _Round:
    """Static device buffers of one (bucket, sampled) round shape, and its graph."""

    def __init__(self, runner, nb: int, sampled: bool):
        model, device = runner.model, runner.device
        w = runner.width
        self.nb, self.sampled = nb, sampled
        self.plan = torch.zeros(3, nb, dtype=torch.int64, device=device)         # slots | counts | round numbers
        self.cu_rows = (torch.arange(nb + 1, device=device) * w).int()
        self.wire = torch.zeros(nb * w + 4 * nb, dtype=torch.int64, device=device)
        self.tokens = torch.zeros(nb, w, dtype=torch.int64, device=device)
        self.retained = torch.zeros(nb, w, model.config.hidden_size, dtype=model.dtype, device=device)
        self.status = torch.zeros(nb, dtype=torch.int32, device=device)
        if sampled:
            vocab = model.config.vocab_size
            self.draft_logits = torch.zeros(nb * w, vocab, dtype=model.dtype, device=device)
            self.workspace = torch.empty(_capi.load().rlt_accept_rejection_workspace_bytes(nb * w),
                                         dtype=torch.uint8, device=device)
        self.graph: torch.cuda.CUDAGraph | None = None


class B200SpeculativeRunner:
    """Block and pipeline self-speculation on the B200 verify-step kernels.

    model: a `LoopedLM` (prelude / recurrent / coda).  cache: an object with `key`, `value` (the
    LAST_EXITED pools `[blocks, layers, block, kv_heads, head_dim]`), `block`, `max_pages`,
    `refcounts` (or None) and `device_tables(request_id) -> int32 [planes, pages]` — `PagedKV`
    here, or an adapter over the reference's `KVCacheManager` allocations.  The host's spans must
    lie inside the pages the cache has reserved for a request on every plane (the reference's
    scheduler reserves them before it schedules a span, core/scheduler.py:747-757).
    """

    def __init__(self, model, cache, config: SpeculativeConfig, *, max_num_seqs: int, cuda_graphs: bool = True,
                 capture_sizes=None, compute_stream=None, report_frontiers: bool = True):
        if config.target_loops > model.config.total_ut_steps:
            raise ValueError("target_loops exceeds the model's recurrent depth")
        self.model, self.cache, self.config = model, cache, config
        self.device = model.device
        self.width = config.num_speculative_tokens + 1 if config.mode == "block" else \
            min(config.num_speculative_tokens + 1, config.target_loops // config.draft_loops)
        self.max_num_seqs = max_num_seqs
        self.cuda_graphs = bool(cuda_graphs)
        if self.cuda_graphs and not model.fused:
            raise ValueError("graph capture needs the fused layer path")
        self.compute_stream = compute_stream
        # True: the protocol of the reference's device-resident runner — tickets carry the device's next positions
        # (`ModelRunnerOutput.frontiers`), from which its scheduler releases the round's placeholders without
        # truncating (core/scheduler.py:1362-1386), and the engine counts deliveries and retires tickets.
        # False: the protocol of its synchronous runner — `frontiers` is None, after which the scheduler calls
        # `truncate_suffix` itself (:1386-1394), and a collected ticket has counted its own delivery.
        self.report_frontiers = report_frontiers
        self.stats = SpeculativeStats()
        self.discarded_rounds = 0          # counters the reference's engine keeps on its runner
        self.readback_waits = 0            # (engine/stage_engine.py:737,747)
        self.states: dict[str, SpeculativeRequestState] = {}
        slots = 2 * max_num_seqs + 1                       # the last slot is the padding rows' dummy
        self.dummy_slot = slots - 1
        self.free_slots = list(reversed(range(slots - 1)))
        planes = model.config.total_ut_steps
        dev = self.device
        self.slot_values = torch.zeros(slots, 2, dtype=torch.int64, device=dev)
        self.slot_tables = torch.zeros(slots, planes, cache.max_pages, dtype=torch.int32, device=dev)
        self.slot_temperature = torch.zeros(slots, dtype=torch.float32, device=dev)
        self.slot_top_k = torch.full((slots,), -1, dtype=torch.int32, device=dev)
        self.slot_top_p = torch.ones(slots, dtype=torch.float32, device=dev)
        self.slot_seed = torch.zeros(slots, dtype=torch.int64, device=dev)
        self.slot_limit = torch.zeros(slots, dtype=torch.int64, device=dev)
        if config.mode == "pipeline":
            w, hidden = self.width, model.config.hidden_size
            self.pipeline = PipelineState(
                tokens=torch.zeros(slots, w, dtype=torch.int64, device=dev),
                depths=torch.zeros(slots, w, dtype=torch.int64, device=dev),
                candidates=torch.zeros(slots, w, dtype=torch.int64, device=dev),
                active=torch.zeros(slots, w, dtype=torch.bool, device=dev),
                hidden=torch.zeros(slots, w, hidden, dtype=model.dtype, device=dev),
                token=torch.zeros(slots, dtype=torch.int64, device=dev),
                position=torch.zeros(slots, dtype=torch.int64, device=dev))
        # Batch sizes a round is padded to.  With graphs every size has its own graph; sizes given
        # explicitly are honoured without graphs too (the eager round then has the graph's shape).
        self.bucketed = self.cuda_graphs or capture_sizes is not None
        if capture_sizes is None:
            capture_sizes = [n for n in (1, 2, 4, 8, 16, 32, 64) if n < max_num_seqs]
            capture_sizes += list(range(96, max_num_seqs, 32)) + [max_num_seqs]
        self.capture_sizes = sorted(set(int(n) for n in capture_sizes if int(n) >= 1))
        if not self.capture_sizes or self.capture_sizes[-1] < max_num_seqs:
            self.capture_sizes.append(max_num_seqs)
        largest = self.capture_sizes[-1] if self.bucketed else max_num_seqs
        self.buffers = [_HostBuffer(3 * largest, max(largest * self.width + 4 * largest, 6 * largest))
                        for _ in range(2)]
        self._rounds: dict[tuple, object] = {}     # (bucket, sampled) -> _Round, ("pipeline", bucket) -> _PipelineRound
        self._pool = None
        self._bootstrap_keepalive: list = []

    # ---- request state ---------------------------------------------------------------------
    def _state(self, request) -> SpeculativeRequestState:
        """The request's device slot; created on its first round from the host's knowledge of the
        request (bootstrap only: afterwards the token and position stay on the device)."""
        rid = request.request_id
        state = self.states.get(rid)
        if state is not None:
            if state.request is not request:
                raise RuntimeError("speculative request state reused before retirement")
            return state
        if not self.free_slots:
            raise RuntimeError("no free speculative slot: release finished requests first")
        slot = self.free_slots.pop()
        p = request.sampling_params
        limit = len(request.prompt_token_ids) + p.max_tokens - 1
        host = torch.tensor([request.input_token_id, request.position, p.seed, limit, p.top_k],
                            dtype=torch.int64).pin_memory()
        host_f = torch.tensor([p.temperature, p.top_p], dtype=torch.float32).pin_memory()
        values = host.to(self.device, non_blocking=True)
        values_f = host_f.to(self.device, non_blocking=True)
        self._bootstrap_keepalive.append((host, host_f))
        self.slot_values[slot].copy_(values[:2])
        self.slot_seed[slot:slot + 1].copy_(values[2:3])
        self.slot_limit[slot:slot + 1].copy_(values[3:4])
        self.slot_top_k[slot:slot + 1].copy_(values[4:5])
        self.slot_temperature[slot:slot + 1].copy_(values_f[0:1])
        self.slot_top_p[slot:slot + 1].copy_(values_f[1:2])
        tables = self.cache.device_tables(rid)
        self.slot_tables[slot].zero_()
        self.slot_tables[slot, :, : tables.shape[1]].copy_(tables)
        if self.config.mode == "pipeline":
            s = self.pipeline
            s.tokens[slot].copy_(values[0:1].expand(self.width))
            s.depths[slot].zero_()
            s.candidates[slot].zero_()
            s.active[slot].zero_()
            s.active[slot, 0] = True
            s.hidden[slot].zero_()
            s.token[slot:slot + 1].copy_(values[0:1])
            s.position[slot:slot + 1].copy_(values[1:2])
        state = SpeculativeRequestState(request, slot)
        self.states[rid] = state
        return state

    def refresh_tables(self, request) -> None:
        """Copy the request's block tables to its slot again (after the cache grew its allocation)."""
        state = self.states.get(request.request_id)
        if state is not None and state.request is request:
            tables = self.cache.device_tables(request.request_id)
            self.slot_tables[state.slot, :, : tables.shape[1]].copy_(tables)

    def request_ready(self, request) -> bool:
        """Whether every round submitted for the request has run (async_speculative.py:663-665)."""
        state = self.states.get(request.request_id)
        return state is None or state.event is None or state.event.query()

    def release(self, request) -> None:
        """Discard this request generation's device state, after its last submitted round has run: the
        caller frees the request's pages next, and another stream may write them (async_speculative.py:667-676)."""
        state = self.states.get(request.request_id)
        if state is None:
            return
        if state.request is not request:
            raise RuntimeError("releasing a different speculative request generation")
        if state.event is not None:
            state.event.synchronize()
        del self.states[request.request_id]
        self.free_slots.append(state.slot)

    def synchronize(self) -> None:
        """Drain the stream the rounds run on (async_speculative.py:689-691)."""
        stream = self.compute_stream if self.compute_stream is not None else torch.cuda.current_stream(self.device)
        stream.synchronize()

    def discard_buffers(self) -> None:
        """Take back every staging buffer after the streams have drained and all tickets are retired, a
        failed submission's included (async_speculative.py:678-687)."""
        for buffer in self.buffers:
            buffer.leased = False

    def snapshot_pipeline(self, request, device):
        """The request's retained pipeline slots as tensors on `device` (speculative.py:280-287 of
        the reference); None when it has no pipeline state."""
        state = self.states.get(request.request_id)
        if self.config.mode != "pipeline" or state is None or state.request is not request:
            return None
        if state.submitted > state.delivered:
            raise RuntimeError("cannot suspend an uncollected pipeline submission")
        s, slot = self.pipeline, state.slot
        return {"request": request,
                **{name: getattr(s, name)[slot].to(device).clone()
                   for name in ("tokens", "depths", "candidates", "active", "hidden", "token", "position")}}

    def restore_pipeline(self, request, snapshot) -> None:
        if snapshot is None:
            return
        if snapshot["request"] is not request or request.request_id in self.states:
            raise RuntimeError("pipeline snapshot belongs to a different request generation")
        state = self._state(request)
        for name in ("tokens", "depths", "candidates", "active", "hidden", "token", "position"):
            getattr(self.pipeline, name)[state.slot].copy_(snapshot[name].to(self.device))
        self.slot_values[state.slot, 0].copy_(self.pipeline.token[state.slot])
        self.slot_values[state.slot, 1].copy_(self.pipeline.position[state.slot])

    # ---- the round -------------------------------------------------------------------------
    def bucket_of(self, n: int) -> int:
        if not self.bucketed:
            return n
        for size in self.capture_sizes:
            if size >= n:
                return size
        raise ValueError(f"a round of {n} requests exceeds max_num_seqs = {self.capture_sizes[-1]}")

    def _round_body(self, r: _Round) -> None:
        """One whole round on the static buffers of `r`: the launch sequence a graph records."""
        model, cache, cfg, w, nb = self.model, self.cache, self.config, self.width, r.nb
        device = self.device
        slots, counts, rounds = r.plan[0], r.plan[1], r.plan[2]
        values = self.slot_values[slots]                               # (input token, position) per request
        starts = values[:, 1].contiguous()
        tables = self.slot_tables[slots]                               # [nb, planes, pages]
        offsets = torch.arange(w, device=device)
        active = counts[:, None] > offsets[None, :]                    # [nb, w]
        positions = torch.where(active, starts[:, None] + offsets[None, :], 0)
        lengths = torch.where(active, positions + 1, 0).int()
        pages, in_page = positions // cache.block, positions % cache.block
        tokens = r.tokens
        tokens.zero_()
        tokens[:, 0] = torch.where(active[:, 0], values[:, 0], 0)
        if r.sampled:
            temperature = self.slot_temperature[slots]
            top_k, top_p = self.slot_top_k[slots], self.slot_top_p[slots]
            u_draft, u_accept, u_final = round_uniforms(self.slot_seed[slots], rounds, w)
            draft_status = torch.zeros(nb, dtype=torch.int32, device=device)
        # draft: one new position per request and offset, loops 0 .. d-1; the depth-d state is retained
        for o in range(w):
            hidden = model.prelude(tokens[:, o])
            column = pages[:, o:o + 1]
            for depth in range(cfg.draft_loops):
                table = tables[:, depth].contiguous()
                blocks = table.gather(1, column).squeeze(1).long()
                hidden = model.recurrent(hidden, positions[:, o].contiguous(), cache.key, cache.value, blocks,
                                         in_page[:, o].contiguous(), table, lengths[:, o].contiguous(),
                                         write_mask=active[:, o].contiguous())
            r.retained[:, o] = hidden
            if o + 1 == w:
                break
            logits = model.coda(hidden)
            if r.sampled:
                r.draft_logits.view(nb, w, -1)[:, o] = logits
                proposed, status = sample_rows(logits, temperature, u_draft[:, o].contiguous(), top_k, top_p)
                draft_status = torch.maximum(draft_status, torch.where(active[:, o + 1], status, 0))
            else:
                proposed = argmax_rows(logits)
            tokens[:, o + 1] = torch.where(active[:, o + 1], proposed, 0).clamp_min(0)
        # verify: all rows, request-major, loops d .. D-1
        hidden = r.retained.view(nb * w, -1)
        flat_positions, flat_lengths = positions.reshape(-1), lengths.reshape(-1)
        flat_in_page, flat_active = in_page.reshape(-1), active.reshape(-1)
        for depth in range(cfg.draft_loops, cfg.target_loops):
            table = tables[:, depth].repeat_interleave(w, 0)
            blocks = table.gather(1, pages.reshape(-1, 1)).squeeze(1).long()
            hidden = model.recurrent(hidden, flat_positions, cache.key, cache.value, blocks, flat_in_page, table,
                                     flat_lengths, write_mask=flat_active)
        logits = model.coda(hidden)
        counts32 = counts.int()
        result = r.wire[: nb * w + 2 * nb]
        if r.sampled:
            accept_rejection(logits, r.draft_logits, r.cu_rows, tokens, starts, temperature, u_accept.reshape(-1),
                             u_final, slots, self.slot_values, result, top_k, top_p, row_counts=counts32,
                             status=r.status, workspace=r.workspace)
            status = torch.maximum(r.status, draft_status)
        else:
            accept_greedy(logits, r.cu_rows, tokens, starts, slots, self.slot_values, result, row_counts=counts32)
            status = r.status                                           # stays zero
        accepted = result[nb * w: nb * w + nb]
        # rollback to start + emitted: the frontier the host commits, refused inside shared pages
        emitted = torch.where(counts > 0, accepted + 1, 0)
        rolled = rollback(starts, emitted, tables, cache.block, refcounts=cache.refcounts)
        r.wire[nb * w + 2 * nb: nb * w + 3 * nb] = status
        r.wire[nb * w + 3 * nb:] = torch.where(counts > 0, rolled.status, 0)

    def _prepare_round(self, nb: int, sampled: bool) -> _Round:
        key = (nb, sampled)
        r = self._rounds.get(key)
        if r is not None:
            return r
        r = _Round(self, nb, sampled)
        r.plan[0].fill_(self.dummy_slot)                                # a round of padding only
        if self.cuda_graphs:
            stream = torch.cuda.current_stream(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(stream)
            with torch.cuda.stream(side):                               # library handles and workspaces exist before capture
                self._round_body(r)
            stream.wait_stream(side)
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            r.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(r.graph, pool=self._pool):
                self._round_body(r)
        self._rounds[key] = r
        return r

    def prepare(self, *, sampled: bool = False, sizes=None) -> None:
        """Capture the round graphs now (an engine does this at start-up, before it serves)."""
        if not self.cuda_graphs:
            return
        for nb in sorted(sizes or self.capture_sizes, reverse=True):    # largest first: scratch is sized once
            if self.config.mode == "pipeline":
                self._prepare_pipeline(self.bucket_of(nb))
            else:
                self._prepare_round(self.bucket_of(nb), sampled)

    def _lease(self) -> _HostBuffer:
        buffer = next((b for b in self.buffers if not b.leased), None)
        if buffer is None:
            raise RuntimeError("speculative buffers exhausted; retire an earlier round")
        return buffer

    @torch.no_grad()
    def submit(self, batch) -> SpeculativeRoundTicket:
        requests = batch.requests
        if not requests or any(span.token_count <= 0 for span in requests):
            raise ValueError("speculative round requires nonempty verification rows")
        if len(requests) > self.max_num_seqs:
            raise ValueError("speculative round exceeds max_num_seqs")
        capacity = self.cache.max_pages * self.cache.block
        for span in requests:
            upper = span.token_start + span.token_count
            if upper > capacity or upper <= 0:
                raise ValueError("speculative round exceeds reserved context")
        buffer = self._lease()
        stream = self.compute_stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream) if stream is not None else _nullcontext():
            states = tuple(self._state(span.request) for span in requests)
            if self.config.mode == "pipeline":
                ticket = self._submit_pipeline(batch, buffer, states)
            else:
                ticket = self._submit_block(batch, buffer, states)
            buffer.done = torch.cuda.Event()
            buffer.done.record(torch.cuda.current_stream(self.device))
        for state in states:
            state.event = buffer.done
        buffer.leased = True
        ticket.keepalive, self._bootstrap_keepalive = self._bootstrap_keepalive, []
        self.stats.rounds += len(requests)
        return ticket

    def _submit_block(self, batch, buffer, states):
        requests, w = batch.requests, self.width
        n = len(requests)
        if any(span.token_count > w for span in requests):
            raise ValueError("a span is longer than num_speculative_tokens + 1")
        nb = self.bucket_of(n)
        sampled = any(span.request.sampling_params.temperature > 0 for span in requests)
        plan = buffer.plan[: 3 * nb].view(3, nb)
        plan[0, :n] = torch.tensor([s.slot for s in states])
        plan[0, n:] = self.dummy_slot
        plan[1, :n] = torch.tensor([span.token_count for span in requests])
        plan[1, n:] = 0
        plan[2, :n] = torch.tensor([s.submitted for s in states])
        plan[2, n:] = 0
        r = self._prepare_round(nb, sampled)
        r.plan.copy_(plan, non_blocking=True)
        if r.graph is not None:
            r.graph.replay()
        else:
            self._round_body(r)
        buffer.wire[: r.wire.numel()].copy_(r.wire, non_blocking=True)
        for state in states:
            state.submitted += 1
        self.stats.drafted_tokens += sum(span.token_count - 1 for span in requests)
        self.stats.verified_rows += sum(span.token_count for span in requests)
        return SpeculativeRoundTicket(self, batch, buffer, states, nb, w, "block")

    # ---- pipeline mode ---------------------------------------------------------------------
    def _pipeline_body(self, r) -> None:
        """The device part of one pipeline step on the static buffers of `r` (what a graph records): every active
        slot of every request advances `draft_loops` loops at its own depth plane, the LM-head argmax of every slot
        is taken, and `pipeline_shift` applies the outcome to the device state (async_speculative.py:502-584 of the
        reference).  Padding requests carry the dummy slot and a width of 0: no active row, no write, no emission."""
        model, cache, cfg, w, n = self.model, self.cache, self.config, self.width, r.nb
        device = self.device
        slots, widths = r.plan[0], r.plan[1].int()
        s = self.pipeline
        local = PipelineState(tokens=s.tokens[slots], depths=s.depths[slots], candidates=s.candidates[slots],
                              active=s.active[slots], hidden=s.hidden[slots], token=s.token[slots],
                              position=s.position[slots])
        tables = self.slot_tables[slots]
        request_of_row = torch.arange(n, device=device).repeat_interleave(w)
        slot_of_row = torch.arange(w, device=device).repeat(n)
        # a span narrower than the pipeline advances only its first slots (async_speculative.py:503-505)
        active = local.active.view(-1) & (slot_of_row < widths[request_of_row])
        depths = local.depths.view(-1)
        positions = torch.where(active, local.position[request_of_row] + slot_of_row, 0)
        hidden = torch.where((depths == 0)[:, None], model.prelude(local.tokens.view(-1)),
                             local.hidden.view(n * w, -1))
        lengths = torch.where(active, positions + 1, 0).int()
        for offset in range(cfg.draft_loops):
            plane = torch.where(active, depths + offset, 0)
            table = tables[request_of_row, plane].contiguous()
            blocks = table.gather(1, (positions // cache.block)[:, None]).squeeze(1).long()
            hidden = model.recurrent(hidden, positions, cache.key, cache.value, blocks, positions % cache.block, table,
                                     lengths, write_mask=active)
        choices = argmax_rows(model.coda(hidden))
        row_starts = (torch.arange(n, device=device) * w).int()
        wire = pipeline_shift(local, widths, row_starts, choices, hidden.contiguous(), self.slot_limit[slots],
                              draft_loops=cfg.draft_loops, target_loops=cfg.target_loops)
        for name in ("tokens", "depths", "candidates", "active", "hidden", "token", "position"):
            getattr(s, name)[slots] = getattr(local, name)
        r.wire.copy_(wire.reshape(-1))

    def _prepare_pipeline(self, nb: int):
        r = self._rounds.get(("pipeline", nb))
        if r is not None:
            return r
        r = _PipelineRound(self, nb)
        r.plan[0].fill_(self.dummy_slot)                                # a step of padding only: changes nothing
        if self.cuda_graphs:
            stream = torch.cuda.current_stream(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(stream)
            with torch.cuda.stream(side):                               # library handles and workspaces exist before capture
                self._pipeline_body(r)
            stream.wait_stream(side)
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            r.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(r.graph, pool=self._pool):
                self._pipeline_body(r)
        self._rounds[("pipeline", nb)] = r
        return r

    def _submit_pipeline(self, batch, buffer, states):
        """One pipeline step: the plan (slots, widths) goes up, the step runs — replayed from the graph of its batch-size
        bucket when graphs are on — and the six-word records come down."""
        w, n = self.width, len(batch.requests)
        if any(span.request.sampling_params.temperature > 0 for span in batch.requests):
            raise ValueError("pipeline speculation supports greedy requests only")
        nb = self.bucket_of(n)
        plan = buffer.plan[: 2 * nb].view(2, nb)
        plan[0, :n] = torch.tensor([s.slot for s in states])
        plan[0, n:] = self.dummy_slot
        plan[1, :n] = torch.tensor([min(span.token_count, w) for span in batch.requests])
        plan[1, n:] = 0
        r = self._prepare_pipeline(nb)
        r.plan.copy_(plan, non_blocking=True)
        if r.graph is not None:
            r.graph.replay()
        else:
            self._pipeline_body(r)
        buffer.wire[: 6 * nb].copy_(r.wire, non_blocking=True)
        for state in states:
            state.submitted += 1
        return SpeculativeRoundTicket(self, batch, buffer, states, n, w, "pipeline")


class _PipelineRound:
    """Static device buffers of one pipeline step shape, and its graph."""

    def __init__(self, runner, nb: int):
        self.nb = nb
        self.plan = torch.zeros(2, nb, dtype=torch.int64, device=runner.device)
        self.wire = torch.zeros(6 * nb, dtype=torch.int64, device=runner.device)
        self.graph = None


class _nullcontext:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False
