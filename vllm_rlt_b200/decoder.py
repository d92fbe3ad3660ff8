"""Greedy self-speculative decoding of a looped LM on the B200 kernels (block mode).

The loop of `SpeculativeRunner._submit_round` / `_collect_round`
(`vllm_rlt/worker/speculative.py:418-511` of the reference) with the reference's round geometry
(a round of request i processes `c_i = min(K+1, max_tokens - generated_i)` input
positions starting at the last committed token; draft offset o runs loops `0..d-1` and proposes
token o+1 from `coda(hidden_d).argmax`; the retained depth-d states of all c_i rows then run
loops `d..D-1` and every row's argmax is a target), on a LAST_EXITED paged KV cache (one plane
per loop depth).  Acceptance, the next token / position and the rollback frontier are computed
on the device by `accept_greedy` / `rollback`; the host reads one small buffer per round.

`native` decoding (one token per step through all loops) is provided for the token-identity
check the reference applies to its own runner (tests/test_speculative.py:71-87 there).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .kv_cache import rollback
from .looped_lm import LoopedLM
from .prefix_cache import PrefixIndex
from .speculative import (PipelineState, accept_greedy, accept_rejection, argmax_rows, pipeline_shift,
                          raise_for_status, sample_rows)


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
    refcounts: torch.Tensor | None = None   # int32 [blocks], holders of every page (prefix reuse only)

    @classmethod
    def allocate(cls, model: LoopedLM, capacities, block: int, *, permute_seed: int | None = 0, prompts=None):
        """Pages for `capacities[i]` tokens of every request on every depth plane.  With `prompts`
        (prefix reuse), request i maps the indexed complete pages of `prompts[i][:-1]` into its
        tables instead of taking fresh ones (`KVCacheManager.allocate(..., prefix=...)`,
        core/kv_cache_manager.py:277-319) and then offers its own complete prompt pages to the
        requests after it; `shared_tokens[i]` is how many leading prompt tokens it does not compute."""
        c = model.config
        planes = c.total_ut_steps
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
        if index is not None:
            index.remap(order.tolist())
        refcounts = None
        if index is not None:
            refcounts = torch.zeros(total, dtype=torch.int32)
            for b, holders in index.refs.items():
                refcounts[b] = holders
            refcounts = refcounts.to(model.device)
        shape = (total, c.num_hidden_layers, block, c.num_key_value_heads, c.head_dim)
        return cls(torch.zeros(shape, device=model.device, dtype=model.dtype),
                   torch.zeros(shape, device=model.device, dtype=model.dtype), tables.to(model.device), block,
                   shared_tokens, index, refcounts)

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
    def __init__(self, model: LoopedLM, *, block: int = 16, cuda_graphs: bool = False, prefix_caching: bool = False):
        self.model = model
        self.block = block
        self.cuda_graphs = cuda_graphs
        self.prefix_caching = prefix_caching   # CacheConfig.enable_prefix_caching of the reference
        self.stats = DecodeStats()
        self._graphs = None

    # ---- shared pieces -------------------------------------------------------------------
    def _upload(self, host_tensors):
        """int64 CPU tensors -> device tensors through one pinned staging buffer and one
        asynchronous copy.  The buffer is reused by the next call, which the decoder makes only
        after it has read a round's results back (so the copy has completed)."""
        sizes = [t.numel() for t in host_tensors]
        total = sum(sizes)
        if getattr(self, "_staging", None) is None or self._staging.numel() < total:
            self._staging = torch.empty(max(total, 4096) * 2, dtype=torch.int64, pin_memory=True)
        torch.cat([t.reshape(-1).long() for t in host_tensors], out=self._staging[:total])
        return self._staging[:total].to(self.model.device, non_blocking=True).split(sizes)

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
            tables = kv.tables[:, depth]
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

    # ---- pipeline self-speculation --------------------------------------------------------
    @torch.no_grad()
    def generate_pipeline(self, prompts, max_tokens: int, *, num_speculative_tokens: int, draft_loops: int = 2,
                          target_loops: int | None = None):
        """Pipeline-mode self-speculation, greedy (`AsyncSpeculativeRunner._pipeline_step`,
        worker/async_speculative.py:502-584 of the reference).

        Every request keeps `width = min(k + 1, D // d)` oldest-first token slots on the device.  A
        step advances every active slot by `d` loops at its own depth plane (slot j sits at
        position `position + j`), takes the LM-head argmax of every slot, and `pipeline_shift`
        applies the outcome: a slot that reached depth d proposes the next token (born at the tail),
        the head slot that reached depth D is emitted and checked against the candidate it was
        drafted from; a mismatch drops its descendants and restarts from the corrected token.  The
        host reads six integers per request and step."""
        model, device = self.model, self.model.device
        target_loops = target_loops or model.config.total_ut_steps
        if not 0 < draft_loops <= target_loops <= model.config.total_ut_steps or target_loops % draft_loops:
            raise ValueError("target_loops must be a positive multiple of draft_loops")
        width = min(num_speculative_tokens + 1, target_loops // draft_loops)
        n = len(prompts)
        kv = self._allocate(prompts, [len(p) + max_tokens + width + 1 for p in prompts])
        first = self._prefill(kv, prompts)
        generated = [[t] for t in first]
        token = torch.tensor(first, device=device)
        state = PipelineState(
            tokens=token[:, None].repeat(1, width).contiguous(),
            depths=torch.zeros(n, width, dtype=torch.int64, device=device),
            candidates=torch.zeros(n, width, dtype=torch.int64, device=device),
            active=(torch.arange(width, device=device) == 0)[None, :].repeat(n, 1).contiguous(),
            hidden=torch.zeros(n, width, model.config.hidden_size, dtype=model.dtype, device=device),
            token=token.clone(),
            position=torch.tensor([len(p) for p in prompts], device=device))
        limits = torch.tensor([len(p) + max_tokens - 1 for p in prompts], device=device)
        widths = torch.full((n,), width, dtype=torch.int32, device=device)
        row_starts = (torch.arange(n, device=device) * width).int()
        request_of_row = torch.arange(n, device=device).repeat_interleave(width)
        slot_of_row = torch.arange(width, device=device).repeat(n)
        for _ in range(max_tokens * (target_loops // draft_loops) + 8):      # each step emits or advances
            if all(len(g) >= max_tokens for g in generated):
                break
            active = state.active.view(-1)
            depths = state.depths.view(-1)
            positions = torch.where(active, state.position[request_of_row] + slot_of_row, 0)
            hidden = torch.where((depths == 0)[:, None], model.prelude(state.tokens.view(-1)),
                                 state.hidden.view(n * width, -1))
            lengths = torch.where(active, positions + 1, 0).int()
            for offset in range(draft_loops):
                plane = torch.where(active, depths + offset, 0)
                tables = kv.tables[request_of_row, plane].contiguous()
                blocks = tables.gather(1, (positions // self.block)[:, None]).squeeze(1).long()
                hidden = model.recurrent(hidden, positions, kv.key, kv.value, blocks, positions % self.block, tables,
                                         lengths, write_mask=active)
            self.stats.loop_passes += draft_loops
            choices = argmax_rows(model.coda(hidden).float().contiguous())
            wire = pipeline_shift(state, widths, row_starts, choices, hidden.contiguous(), limits,
                                  draft_loops=draft_loops, target_loops=target_loops)
            for i, (prediction, accepted, emitted, _, drafted, verified) in enumerate(wire.tolist()):  # the step's one host read
                if emitted and len(generated[i]) < max_tokens:
                    generated[i].append(prediction)
                    self.stats.committed_tokens += 1
                    self.stats.accepted_tokens += accepted
                self.stats.drafted_tokens += drafted
                self.stats.verified_rows += verified
            self.stats.rounds += n
        return [g[:max_tokens] for g in generated]

    # ---- block self-speculation ----------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts, max_tokens: int, *, num_speculative_tokens: int, draft_loops: int = 2,
                 target_loops: int | None = None, temperature: float = 0.0, top_k: int = -1, top_p: float = 1.0,
                 seed: int = 0, after_prefill=None):
        """Block self-speculation.  `temperature == 0` is greedy acceptance; otherwise drafts are
        sampled from the draft distribution (softmax(draft logits / T) after top-k / top-p, as
        Sampler.probabilities builds it) and verified by rejection sampling with residual
        resampling (worker/speculative.py:47-63, 483-510 of the reference), with every uniform
        drawn from one seeded device generator in the reference's order per round: the draft
        draws, then the accept tests, then the final (residual or bonus) draw.  `after_prefill`, if
        given, is called once the prompts are in the cache (benchmarks start their clock there)."""
        model, device = self.model, self.model.device
        sampled = temperature > 0
        generator = torch.Generator(device=device).manual_seed(seed) if sampled else None
        if not 0 < top_p <= 1 or (top_k != -1 and top_k < 1):
            raise ValueError("top_p must be in (0, 1] and top_k must be -1 or positive")
        filtered = sampled and (top_k > 0 or top_p < 1)

        def filters(count):
            if not filtered:
                return None, None
            return (torch.full((count,), top_k, dtype=torch.int32, device=device),
                    torch.full((count,), top_p, dtype=torch.float32, device=device))
        target_loops = target_loops or model.config.total_ut_steps
        if not 0 < draft_loops < target_loops <= model.config.total_ut_steps:
            raise ValueError("draft_loops must be smaller than target_loops")
        k = num_speculative_tokens
        kv = self._allocate(prompts, [len(p) + max_tokens + k + 1 for p in prompts])
        generated = [[t] for t in self._prefill(kv, prompts)]  # the first token is the prefill's argmax
        if self.cuda_graphs:
            self._graphs = GraphedLoops(model, kv)
            self._graphs.prepare(len(prompts) * (k + 1))
        if after_prefill is not None:
            after_prefill()
        slot_values = torch.zeros(len(prompts), 2, dtype=torch.int64, device=device)
        while any(len(g) < max_tokens for g in generated):
            active = [i for i, g in enumerate(generated) if len(g) < max_tokens]
            counts = [min(k + 1, max_tokens - len(generated[i])) for i in active]
            starts = [len(prompts[i]) + len(generated[i]) - 1 for i in active]
            n, width = len(active), max(counts)
            rows_total = sum(counts)
            counts_t = torch.tensor(counts)
            # which (request, offset) cells exist, and where each lands among the retained rows
            present = counts_t[:, None] > torch.arange(width)[None, :]                 # [n, width]
            per_offset = present.sum(0)                                                # rows of draft pass o
            rank = present.long().cumsum(0) - 1                                        # row of request j in pass o
            base = torch.cat([torch.zeros(1, dtype=torch.long), per_offset.cumsum(0)[:-1]])
            firsts = [0] + counts_t.cumsum(0).tolist()[:-1]
            in_pass_host = [present[:, o].nonzero().flatten() for o in range(width)]
            drafting_host = [present[present[:, o], o + 1].nonzero().flatten() if o + 1 < width
                             else torch.zeros(0, dtype=torch.long) for o in range(width)]
            row_request = torch.repeat_interleave(torch.arange(n), counts_t)
            row_offset = torch.cat([torch.arange(c) for c in counts])
            # every index tensor of the round goes to the device in one pinned, asynchronous copy:
            # a pageable upload in the middle of a round would wait for the GPU and stall the launches
            (active_t, starts_t, last_t, gather, first_row, row_request_t, row_offset_t, cu_rows64, *per_pass) = \
                self._upload([torch.tensor(active), torch.tensor(starts),
                              torch.tensor([generated[i][-1] for i in active]), (base[None, :] + rank)[present],
                              torch.tensor(firsts), row_request, row_offset,
                              torch.tensor([0] + counts_t.cumsum(0).tolist()), *in_pass_host, *drafting_host])
            in_pass_dev, drafting_dev = per_pass[:width], per_pass[width:]
            tokens = torch.zeros(n, width, dtype=torch.int64, device=device)
            tokens[:, 0] = last_t
            draft_logits = None
            if sampled:  # row j of a request keeps the logits its draft j+1 was sampled from
                draft_logits = torch.zeros(rows_total, model.config.vocab_size, dtype=torch.float32, device=device)
                u_draft = torch.rand(n, width, generator=generator, device=device)
            retained = []
            # draft: one new position per request and offset, loops 0 .. d-1
            for offset in range(width):
                in_pass = in_pass_dev[offset]                                           # requests with c > offset
                hidden = model.prelude(tokens[in_pass, offset])
                for depth in range(draft_loops):
                    hidden = self._loop(kv, hidden, active_t[in_pass], starts_t[in_pass] + offset, depth)
                self.stats.loop_passes += draft_loops
                self.stats.context_tokens_read += draft_loops * sum(s + offset + 1 for s, c in zip(starts, counts) if c > offset)
                retained.append(hidden)
                if offset + 1 >= width:
                    break
                drafting = drafting_dev[offset]                                         # rows of this pass that draft on
                if drafting.numel() == 0:
                    break
                drafting_requests = in_pass[drafting]
                logits = model.coda(hidden[drafting]).float().contiguous()
                if sampled:
                    draft_logits[first_row[drafting_requests] + offset] = logits
                    proposed, _ = sample_rows(logits, torch.full((logits.shape[0],), temperature, device=device),
                                              u_draft[drafting_requests, offset].contiguous(), *filters(logits.shape[0]))
                else:
                    proposed = argmax_rows(logits)
                tokens[drafting_requests, offset + 1] = proposed
                self.stats.drafted_tokens += int(logits.shape[0])
                self.stats.coda_rows += int(logits.shape[0])
            # verify: the retained depth-d states of all rows, request-major, loops d .. D-1
            hidden = torch.cat(retained)[gather]
            requests = active_t[row_request_t]
            positions = starts_t[row_request_t] + row_offset_t
            for depth in range(draft_loops, target_loops):
                hidden = self._loop(kv, hidden, requests, positions, depth)
            self.stats.loop_passes += target_loops - draft_loops
            self.stats.context_tokens_read += (target_loops - draft_loops) * sum(s + c for s, c in zip(starts, counts))
            self.stats.coda_rows += rows_total
            logits = model.coda(hidden).float().contiguous()
            cu_rows = cu_rows64.int()
            start_tensor = starts_t
            slots = torch.arange(n, device=device)
            if sampled:
                result, status = accept_rejection(
                    logits, draft_logits, cu_rows, tokens.contiguous(), start_tensor,
                    torch.full((n,), temperature, device=device), torch.rand(rows_total, generator=generator, device=device),
                    torch.rand(n, generator=generator, device=device), slots, slot_values[:n].contiguous(),
                    None, *filters(n))
            else:
                status = torch.zeros(n, dtype=torch.int32, device=device)
                result = accept_greedy(logits, cu_rows, tokens.contiguous(), start_tensor, slots,
                                       slot_values[:n].contiguous())
            accepted = result[rows_total:rows_total + n]
            # with prefix reuse the page reference counts go along: a frontier inside a shared page is refused
            rolled = rollback(start_tensor, accepted + 1, kv.tables[active_t].contiguous(), self.block,
                              refcounts=kv.refcounts)
            values = torch.cat([result, rolled.frontier, status.long(), rolled.status.long()]).tolist()  # the round's one host read
            if kv.refcounts is not None and 4 in values[len(values) - n:]:
                raise RuntimeError("rollback refused: the frontier of a request lies in a shared page")
            values = values[:len(values) - n]
            raise_for_status(values[rows_total + 3 * n:])
            for j, i in enumerate(active):
                a = values[rows_total + j]
                emitted = values[firsts[j]:firsts[j] + a + 1]
                generated[i].extend(emitted)
                assert values[rows_total + n + j] == starts[j] + a + 1 == values[rows_total + 2 * n + j]
                self.stats.accepted_tokens += a
                self.stats.committed_tokens += len(emitted)
            self.stats.rounds += n
            self.stats.verified_rows += rows_total
        self._graphs = None
        return [g[:max_tokens] for g in generated]
