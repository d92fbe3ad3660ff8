"""Self-speculative decoding of a looped LM on the B200 kernels: the engine loop around the runner.

`SelfSpeculativeDecoder` plays the part of the reference's engine for this path
(`StageEngine._step_async_speculative`, `vllm_rlt/engine/stage_engine.py:732-793`, with the span
rule of `Scheduler._make_scheduled_request`, `vllm_rlt/core/scheduler.py:603-608`): it reserves the
pages, runs the prompts, schedules spans `(request, token_start, token_count = min(K + 1, remaining))`
on a LAST_EXITED paged KV cache (one plane per loop depth), submits them to
`B200SpeculativeRunner`, keeps up to two rounds in flight, and applies the collected results
(tokens, frontier check) the way `Scheduler.update_from_output` does (`:1360-1397`).  All of the
round itself — draft and verify passes, acceptance, device state, rollback — is the runner's.

`native` decoding (one token per step through all loops) is provided for the token-identity
check the reference applies to its own runner (tests/test_speculative.py:71-87 there).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from collections import deque

from .looped_lm import LoopedLM
from .prefix_cache import PrefixIndex
from .runner import (B200SpeculativeRunner, Request, SamplingParams, ScheduledRequest, SchedulerOutput,
                     SpeculativeConfig)
from .speculative import argmax_rows


@dataclass
class DecodeStats:
    """Counters of the reference's SpeculativeStats (worker/speculative.py:23-29)."""

    rounds: int = 0
    drafted_tokens: int = 0
    accepted_tokens: int = 0
    committed_tokens: int = 0
    verified_rows: int = 0
    # work accounting of the decode loop (not in the reference): recurrent passes over all layers,
    # context tokens whose K/V those passes had to read (once per request and pass), LM-head rows
    loop_passes: int = 0
    context_tokens_read: int = 0
    prefix_hit_tokens: int = 0          # prompt tokens mapped from the prefix index (KVCacheManager.prefix_hits)
    prompt_tokens_computed: int = 0
    coda_rows: int = 0


@dataclass
class PagedKV:
    """A LAST_EXITED paged pool: `[blocks, layers, block, kv_heads, head_dim]` K and V, and one block
    table per (request, depth plane), `tables[n, planes, pages]` (core/kv_cache_manager.py:135-145)."""

    key: torch.Tensor
    value: torch.Tensor
    tables: torch.Tensor
    block: int
    shared_tokens: list | None = None   # per request: leading prompt tokens mapped from the prefix index
    prefix_index: PrefixIndex | None = None
    refcounts: torch.Tensor | None = None   # int32 [blocks], holders of every page (prefix reuse; always present in a reserved pool)
    reserved: bool = False                  # built by `reserve`: tables and holders are rewritten in place by `assign`

    @staticmethod
    def _plan_tables(planes: int, capacities, block: int, permute_seed, prompts):
        """Page ids for `capacities[i]` tokens of every request on every depth plane: int32 tables
        `[requests, planes, pages]` (padding -1), the number of pages they name, and with `prompts`
        (prefix reuse) the tokens every request maps instead of computing, the index and the holders."""
        pages = [-(-n // block) for n in capacities]
        width = max(pages)
        index = PrefixIndex(block) if prompts is not None else None
        logical = torch.full((len(capacities), planes, width), -1, dtype=torch.int64)
        shared_tokens = []
        cursor = 0
        for i, n in enumerate(pages):
            prefix = index.lookup(prompts[i]) if index is not None else ()
            hit = len(prefix)
            shared_tokens.append(hit * block)
            for plane in range(planes):
                for j in range(hit):
                    logical[i, plane, j] = prefix[j][plane]
                logical[i, plane, hit:n] = torch.arange(cursor, cursor + n - hit)
                cursor += n - hit
            if index is not None:
                index.claim(prefix)
                index.own(logical[i, :, hit:n].reshape(-1).tolist())
                index.publish(prompts[i], len(prompts[i]), logical[i].tolist())
        total = cursor
        order = torch.arange(total, dtype=torch.int64)
        if permute_seed is not None:  # physical pages deliberately out of order
            order = order[torch.randperm(total, generator=torch.Generator().manual_seed(permute_seed))]
        tables = torch.where(logical >= 0, order[logical.clamp_min(0)], logical).to(torch.int32)
        holders = None
        if index is not None:
            index.remap(order.tolist())
            holders = index.refs
        return tables, total, shared_tokens, index, holders

    @classmethod
    def allocate(cls, model: LoopedLM, capacities, block: int, *, permute_seed: int | None = 0, prompts=None):
        """A pool of exactly the pages `capacities[i]` tokens of every request need on every depth plane.
        With `prompts` (prefix reuse), request i maps the indexed complete pages of `prompts[i][:-1]` into
        its tables instead of taking fresh ones (`KVCacheManager.allocate(..., prefix=...)`,
        core/kv_cache_manager.py:277-319) and then offers its own complete prompt pages to the requests
        after it; `shared_tokens[i]` is how many leading prompt tokens it does not compute."""
        c = model.config
        tables, total, shared_tokens, index, holders = cls._plan_tables(c.total_ut_steps, capacities, block,
                                                                        permute_seed, prompts)
        kv = cls.reserve(model, total, len(capacities), tables.shape[2], block)
        kv.reserved, kv.refcounts = False, None
        kv._install(tables, total, shared_tokens, index, holders)
        return kv

    @classmethod
    def reserve(cls, model: LoopedLM, pages: int, requests: int, width: int, block: int):
        """An engine's fixed pool: `pages` physical pages, tables for up to `requests` requests of up to
        `width` pages per plane.  `assign` hands the pages out to a set of requests; the pool, and therefore
        every pointer a captured round graph holds, stays where it is from one set of requests to the next."""
        c = model.config
        shape = (pages, c.num_hidden_layers, block, c.num_key_value_heads, c.head_dim)
        return cls(torch.zeros(shape, device=model.device, dtype=model.dtype),
                   torch.zeros(shape, device=model.device, dtype=model.dtype),
                   torch.full((requests, c.total_ut_steps, width), -1, dtype=torch.int32, device=model.device), block,
                   refcounts=torch.zeros(pages, dtype=torch.int32, device=model.device), reserved=True)

    def assign(self, capacities, *, permute_seed: int | None = 0, prompts=None):
        """Hands the pool's pages out afresh to requests of the given capacities (rows 0..n-1 of the tables).
        What earlier requests left in the pages is never read: a request writes a position before any row
        attends to it."""
        tables, total, shared_tokens, index, holders = self._plan_tables(self.tables.shape[1], capacities, self.block,
                                                                         permute_seed, prompts)
        if len(capacities) > self.tables.shape[0] or tables.shape[2] > self.tables.shape[2] or total > self.key.shape[0]:
            raise ValueError(f"{len(capacities)} requests / {tables.shape[2]} pages per plane / {total} pages do not fit "
                             f"the reserved {tuple(self.tables.shape[::2])} tables and {self.key.shape[0]} pages")
        self._install(tables, total, shared_tokens, index, holders)

    def _install(self, tables, total, shared_tokens, index, holders):
        self.tables.fill_(-1)
        self.tables[: tables.shape[0], :, : tables.shape[2]] = tables.to(self.tables.device)
        self.shared_tokens, self.prefix_index = shared_tokens, index
        if holders is None and not self.reserved:
            self.refcounts = None
            return
        counts = torch.zeros(self.key.shape[0], dtype=torch.int32)
        for page, count in (holders or {}).items():
            counts[page] = count
        if self.refcounts is None:
            self.refcounts = counts.to(self.tables.device)
        else:
            self.refcounts.copy_(counts)    # in place: a captured round graph holds this tensor's address

    @property
    def max_pages(self) -> int:
        return self.tables.shape[2]

    def device_tables(self, request_id) -> torch.Tensor:
        """int32 [planes, pages] of one request (requests are named by their row, as a string or int)."""
        return self.tables[int(request_id)]

    def addressing(self, requests: torch.Tensor, positions: torch.Tensor, plane: int):
        """Write addresses, per-row block tables and context lengths of rows (request, position)."""
        tables = self.tables[requests, plane]
        blocks = tables.gather(1, (positions // self.block)[:, None]).squeeze(1).long()
        return blocks, positions % self.block, tables.contiguous(), (positions + 1).int()


class GraphedLoops:
    """One recurrent loop (all layers) as a CUDA graph per row-count bucket.

    The reference captures its decode passes the same way (`worker/cuda_graph.py:338-404`):
    static input buffers, batch sizes rounded up to a bucket, padding rows that neither write
    K/V (they lie at or beyond `active_rows`) nor read any (context length 0, so the attention
    plan gives them no work and zeros as output).  Row grouping is planned on the device inside
    the graph, so a replay follows whatever tables and lengths the buffers hold.
    """

    def __init__(self, model: LoopedLM, kv: PagedKV, *, granularity: int = 64):
        if not model.fused:
            raise ValueError("graph capture needs the fused layer path")
        self.model, self.kv, self.granularity = model, kv, granularity
        self.pool = torch.cuda.graph_pool_handle()
        self.graphs = {}

    def _capture(self, bucket: int):
        model, kv, device = self.model, self.kv, self.model.device
        buffers = dict(
            hidden=torch.zeros(bucket, model.config.hidden_size, dtype=model.dtype, device=device),
            positions=torch.zeros(bucket, dtype=torch.int64, device=device),
            blocks=torch.zeros(bucket, dtype=torch.int64, device=device),
            offsets=torch.zeros(bucket, dtype=torch.int64, device=device),
            tables=torch.zeros(bucket, kv.tables.shape[2], dtype=torch.int32, device=device),
            lengths=torch.zeros(bucket, dtype=torch.int32, device=device),
            active=torch.zeros((), dtype=torch.int32, device=device))

        def run():
            return model._recurrent_fused(buffers["hidden"], buffers["positions"], kv.key, kv.value, buffers["blocks"],
                                          buffers["offsets"], buffers["tables"], buffers["lengths"],
                                          active_rows=buffers["active"])

        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):                      # library handles and workspaces exist before capture
            run()
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self.pool):
            buffers["out"] = run()
        self.graphs[bucket] = (graph, buffers)
        return self.graphs[bucket]

    def bucket_of(self, rows: int) -> int:
        return -(-rows // self.granularity) * self.granularity

    def prepare(self, max_rows: int):
        """Capture every bucket up to `max_rows` now (benchmarks do this before their clock starts)."""
        for bucket in range(self.bucket_of(max_rows), 0, -self.granularity):   # largest first: scratch is sized once
            if bucket not in self.graphs:
                self._capture(bucket)

    def __call__(self, hidden, positions, blocks, offsets, tables, lengths):
        rows = hidden.shape[0]
        graph, b = self.graphs.get(self.bucket_of(rows)) or self._capture(self.bucket_of(rows))
        b["hidden"][:rows] = hidden
        b["positions"][:rows] = positions
        b["blocks"][:rows] = blocks
        b["offsets"][:rows] = offsets
        b["tables"][:rows] = tables
        b["lengths"][:rows] = lengths
        b["lengths"][rows:] = 0
        b["active"].fill_(rows)
        graph.replay()
        return b["out"][:rows].clone()


class SelfSpeculativeDecoder:
    def __init__(self, model: LoopedLM, *, block: int = 16, cuda_graphs: bool = False, prefix_caching: bool = False,
                 capture_sizes=None):
        self.model = model
        self.block = block
        self.cuda_graphs = cuda_graphs
        self.capture_sizes = capture_sizes         # batch sizes with a round graph (None: the runner's default)
        self.runner = None
        self.prefix_caching = prefix_caching   # CacheConfig.enable_prefix_caching of the reference
        self.stats = DecodeStats()
        self._graphs = None

    # ---- shared pieces -------------------------------------------------------------------
    def _loop(self, kv: PagedKV, hidden, requests, positions, depth):
        blocks, offsets, tables, lengths = kv.addressing(requests, positions, depth)
        if self._graphs is not None and self._graphs.kv is kv:
            return self._graphs(hidden, positions, blocks, offsets, tables, lengths)
        return self.model.recurrent(hidden, positions, kv.key, kv.value, blocks, offsets, tables, lengths)

    def _allocate(self, prompts, capacities):
        return PagedKV.allocate(self.model, capacities, self.block, prompts=prompts if self.prefix_caching else None)

    def _prefill(self, kv: PagedKV, prompts):
        """All prompt positions through every loop, packed (one table row per prompt, causal inside
        it); returns the first generated token of each request.  Leading tokens whose pages a request
        shares with an earlier one are not computed: its rows start behind them and attend to the
        shared pages, which the earlier request's rows write in the same pass (within a layer every
        K/V row is written before any row attends)."""
        device = self.model.device
        skips = kv.shared_tokens if kv.shared_tokens is not None else [0] * len(prompts)
        lengths = [len(p) for p in prompts]
        new = [n - s for n, s in zip(lengths, skips)]
        self.stats.prefix_hit_tokens += sum(skips)
        self.stats.prompt_tokens_computed += sum(new)
        requests = torch.tensor([i for i, n in enumerate(new) for _ in range(n)], device=device)
        positions = torch.tensor([j for n, s in zip(lengths, skips) for j in range(s, n)], device=device)
        tokens = torch.tensor([t for p, s in zip(prompts, skips) for t in p[s:]], device=device)
        cu = torch.tensor([0] + torch.tensor(new).cumsum(0).tolist(), dtype=torch.int32, device=device)
        context = torch.tensor(lengths, dtype=torch.int32, device=device)
        hidden = self.model.prelude(tokens)
        for depth in range(self.model.config.total_ut_steps):
            tables = kv.tables[: len(prompts), depth]       # a reserved pool may have more table rows than requests
            blocks = tables[requests].gather(1, (positions // self.block)[:, None]).squeeze(1).long()
            hidden = self.model.recurrent(hidden, positions, kv.key, kv.value, blocks, positions % self.block,
                                          tables.contiguous(), context, packed=(cu, max(new)))
        last = (cu[1:] - 1).long()
        return argmax_rows(self.model.coda(hidden[last]).float().contiguous()).tolist()

    # ---- native decoding -----------------------------------------------------------------
    @torch.no_grad()
    def generate_native(self, prompts, max_tokens: int):
        device = self.model.device
        kv = self._allocate(prompts, [len(p) + max_tokens for p in prompts])
        generated = [[t] for t in self._prefill(kv, prompts)]
        while any(len(g) < max_tokens for g in generated):
            active = [i for i, g in enumerate(generated) if len(g) < max_tokens]
            requests = torch.tensor(active, device=device)
            positions = torch.tensor([len(prompts[i]) + len(generated[i]) - 1 for i in active], device=device)
            hidden = self.model.prelude(torch.tensor([generated[i][-1] for i in active], device=device))
            for depth in range(self.model.config.total_ut_steps):
                hidden = self._loop(kv, hidden, requests, positions, depth)
            for i, token in zip(active, argmax_rows(self.model.coda(hidden).float().contiguous()).tolist()):
                generated[i].append(token)
        return generated

    # ---- self-speculation through the runner ---------------------------------------------
    def _requests(self, prompts, first_tokens, max_tokens, temperature, top_k, top_p, seed):
        return [Request(str(i), list(p), SamplingParams(max_tokens=max_tokens, temperature=temperature, top_k=top_k,
                                                        top_p=top_p, seed=(seed * 1000003 + i) % (2 ** 63)),
                        generated_token_ids=[t])
                for i, (p, t) in enumerate(zip(prompts, first_tokens))]

    def _schedule(self, requests, k: int, pipeline: bool):
        """The speculative spans of one submission (core/scheduler.py:603-608, 734-739 of the reference): at
        most two rounds of a request in flight, `token_count = min(K + 1, remaining)` with the tokens of
        uncollected rounds counted as placeholders, `token_start` the position those placeholders imply."""
        spans = []
        for request in requests:
            if request.finished or request.num_speculative_rounds >= 2:
                continue
            remaining = request.sampling_params.max_tokens - request.num_scheduled_outputs
            if remaining <= 0:
                continue
            spans.append(ScheduledRequest(request, request.position, min(k + 1, remaining)))
        return SchedulerOutput("speculative", spans) if spans else None

    @staticmethod
    def _after_submission(batch, pipeline: bool):
        """`Scheduler.update_after_submission` (core/scheduler.py:1400-1420): the submitted span's tokens
        become placeholders.  Only now, because the runner's first sight of a request reads its committed
        position."""
        for span in batch.requests:
            span.request.num_output_placeholders += 1 if pipeline else span.token_count
            span.request.num_speculative_rounds += 1

    def _apply(self, ticket, output, pipeline: bool, config):
        """`Scheduler.update_from_output` for a speculative round (core/scheduler.py:1360-1397): release
        the placeholders, check the device's frontier against the committed prefix, record the tokens."""
        d, target = config.draft_loops, config.target_loops
        for span, result, frontier in zip(ticket.batch.requests, output.speculative, output.frontiers):
            request = span.request
            request.num_output_placeholders -= 1 if pipeline else span.token_count
            request.num_speculative_rounds -= 1
            if request.finished:
                continue                                     # a round that was in flight when the request ended
            expected = len(request.prompt_token_ids) + len(request.generated_token_ids) - 1
            if frontier != expected + len(result.token_ids):
                raise RuntimeError("speculative GPU frontier disagrees with committed prefix")
            if not pipeline:                                 # work accounting of the round, from the true start
                start, count = expected, span.token_count
                self.stats.context_tokens_read += d * sum(start + o + 1 for o in range(count)) \
                    + (target - d) * (start + count)
            room = request.sampling_params.max_tokens - len(request.generated_token_ids)
            emitted = result.token_ids[:room]
            request.generated_token_ids.extend(emitted)
            self.stats.committed_tokens += len(emitted)
            self.stats.accepted_tokens += min(result.accepted_count, len(emitted))
            if len(request.generated_token_ids) >= request.sampling_params.max_tokens:
                request.finished = True

    def _drive(self, runner, requests, k: int, in_flight: int):
        session = DecodeSession(self, runner, requests, k, in_flight)
        session.run()
        session.close()

    @torch.no_grad()
    def generate_pipeline(self, prompts, max_tokens: int, *, num_speculative_tokens: int, draft_loops: int = 2,
                          target_loops: int | None = None, in_flight: int = 1):
        """Pipeline-mode self-speculation, greedy (`AsyncSpeculativeRunner._pipeline_step`,
        worker/async_speculative.py:502-584 of the reference).

        Every request keeps `width = min(k + 1, D // d)` oldest-first token slots on the device.  A
        step advances every active slot by `d` loops at its own depth plane (slot j sits at
        position `position + j`), takes the LM-head argmax of every slot, and `pipeline_shift`
        applies the outcome: a slot that reached depth d proposes the next token (born at the tail),
        the head slot that reached depth D is emitted and checked against the candidate it was
        drafted from; a mismatch drops its descendants and restarts from the corrected token.  The
        host reads six integers per request and step."""
        model = self.model
        target_loops = target_loops or model.config.total_ut_steps
        if not 0 < draft_loops < target_loops <= model.config.total_ut_steps or target_loops % draft_loops:
            raise ValueError("target_loops must be a multiple of draft_loops and larger than it")
        config = SpeculativeConfig(num_speculative_tokens, draft_loops, target_loops, mode="pipeline")
        width = min(num_speculative_tokens + 1, target_loops // draft_loops)
        kv = self._allocate(prompts, [len(p) + max_tokens + width + 1 for p in prompts])
        requests = self._requests(prompts, self._prefill(kv, prompts), max_tokens, 0.0, -1, 1.0, 0)
        runner = B200SpeculativeRunner(model, kv, config, max_num_seqs=len(prompts), cuda_graphs=self.cuda_graphs,
                                       capture_sizes=self.capture_sizes)
        self.runner = runner
        self._drive(runner, requests, num_speculative_tokens, in_flight)
        return [r.generated_token_ids[:max_tokens] for r in requests]

    @torch.no_grad()
    def open(self, prompts, max_tokens: int, *, num_speculative_tokens: int, draft_loops: int = 2,
             target_loops: int | None = None, temperature: float = 0.0, top_k: int = -1, top_p: float = 1.0,
             seed: int = 0, in_flight: int = 1, kv: PagedKV | None = None,
             runner: B200SpeculativeRunner | None = None) -> "DecodeSession":
        """Everything `generate` does before its first round — pages reserved, prompts run, requests
        created, runner built and (with CUDA graphs) its round graphs captured — as a `DecodeSession`.
        An engine that serves one set of requests after another passes its reserved pool (`PagedKV.reserve`)
        and the runner it built over that pool: the pages are handed out afresh, the runner and its graphs
        are reused."""
        model = self.model
        if not 0 < top_p <= 1 or (top_k != -1 and top_k < 1):
            raise ValueError("top_p must be in (0, 1] and top_k must be -1 or positive")
        target_loops = target_loops or model.config.total_ut_steps
        if not 0 < draft_loops < target_loops <= model.config.total_ut_steps:
            raise ValueError("draft_loops must be smaller than target_loops")
        k = num_speculative_tokens
        config = SpeculativeConfig(k, draft_loops, target_loops)
        capacities = [len(p) + max_tokens + k + 1 for p in prompts]
        if kv is None:
            kv = self._allocate(prompts, capacities)
        else:
            kv.assign(capacities, prompts=prompts if self.prefix_caching else None)
        requests = self._requests(prompts, self._prefill(kv, prompts), max_tokens, temperature, top_k, top_p, seed)
        if runner is None:
            runner = B200SpeculativeRunner(model, kv, config, max_num_seqs=len(prompts), cuda_graphs=self.cuda_graphs,
                                           capture_sizes=self.capture_sizes)
        elif runner.cache is not kv or runner.config != config or runner.max_num_seqs < len(prompts) or runner.states:
            raise ValueError("the runner was built for another pool or configuration, is too small, or still holds requests")
        self.runner = runner
        if runner.cuda_graphs:
            runner.prepare(sampled=temperature > 0)
        return DecodeSession(self, runner, requests, k, in_flight)

    @torch.no_grad()
    def generate(self, prompts, max_tokens: int, *, num_speculative_tokens: int, draft_loops: int = 2,
                 target_loops: int | None = None, temperature: float = 0.0, top_k: int = -1, top_p: float = 1.0,
                 seed: int = 0, after_prefill=None, in_flight: int = 1):
        """Block self-speculation.  `temperature == 0` is greedy acceptance; otherwise drafts are
        sampled from the draft distribution (softmax(draft logits / T) after top-k / top-p, as
        Sampler.probabilities builds it) and verified by rejection sampling with residual
        resampling (worker/speculative.py:47-63, 483-510 of the reference); request i draws from its
        own stream, seeded `seed * 1000003 + i`.  `in_flight = 1` collects a round before the next is
        submitted (the schedule of the reference's synchronous runner, so its counters are
        reproduced); `in_flight = 2` submits the next round first, as the reference's asynchronous
        engine does — the tokens are the same, rounds near a request's output limit are scheduled
        more cautiously.  `after_prefill`, if given, is called once the prompts are in the cache and
        the round graphs exist (benchmarks start their clock there)."""
        session = self.open(prompts, max_tokens, num_speculative_tokens=num_speculative_tokens, draft_loops=draft_loops,
                            target_loops=target_loops, temperature=temperature, top_k=top_k, top_p=top_p, seed=seed,
                            in_flight=in_flight)
        if after_prefill is not None:
            after_prefill()
        session.run()
        session.close()
        return [r.generated_token_ids[:max_tokens] for r in session.requests]


class DecodeSession:
    """The engine loop over one set of requests, one submission or collection at a time (so that a
    caller can time a window of rounds): `submit_round()` schedules and submits the next round if the
    in-flight limit and the requests allow one, `collect_round()` waits for the oldest round and applies
    its tokens, `run()` alternates them until every request has its tokens."""

    def __init__(self, decoder: SelfSpeculativeDecoder, runner: B200SpeculativeRunner, requests, k: int,
                 in_flight: int = 1):
        if in_flight not in (1, 2):
            raise ValueError("one or two rounds in flight")
        self.decoder, self.runner, self.requests, self.k, self.in_flight = decoder, runner, requests, k, in_flight
        self.pipeline = runner.config.mode == "pipeline"
        self.pending = deque()

    def submit_round(self) -> bool:
        if len(self.pending) >= self.in_flight:
            return False
        batch = self.decoder._schedule(self.requests, self.k, self.pipeline)
        if batch is None:
            return False
        self.pending.append(self.runner.submit(batch))
        self.decoder._after_submission(batch, self.pipeline)
        stats, config = self.decoder.stats, self.runner.config
        if self.pipeline:
            stats.loop_passes += config.draft_loops
        else:
            stats.loop_passes += config.draft_loops * max(s.token_count for s in batch.requests) \
                + config.target_loops - config.draft_loops
            stats.coda_rows += sum(2 * s.token_count - 1 for s in batch.requests)
        return True

    def collect_round(self) -> bool:
        if not self.pending:
            return False
        ticket = self.pending.popleft()
        output = ticket.collect()
        if self.runner.report_frontiers:          # the engine's share of the device-resident protocol
            for state, round_id in zip(ticket.states, ticket.rounds):      # (engine/stage_engine.py:738-752)
                if state.delivered != round_id:
                    raise RuntimeError("out-of-order speculative round delivery")
                state.delivered += 1
        self.decoder._apply(ticket, output, self.pipeline, self.runner.config)
        ticket.retire()
        self._sync_stats()
        return True

    def _sync_stats(self):
        stats, source = self.decoder.stats, self.runner.stats
        stats.rounds, stats.drafted_tokens, stats.verified_rows = source.rounds, source.drafted_tokens, source.verified_rows

    def run(self):
        while True:
            while self.submit_round():
                pass
            if not self.collect_round():
                break

    def drain(self):
        while self.collect_round():
            pass

    def close(self):
        self.drain()
        for request in self.requests:
            self.runner.release(request)
        self._sync_stats()
