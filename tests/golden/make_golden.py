"""Generate the golden vectors in this folder by running the vllm-rlt reference itself.

Run once, in a container where the reference checkout is importable:

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

The outputs (``*.pt``: dicts of small CPU tensors / python scalars) are committed; the
tests load them and never import the reference.  Every case records the seeded inputs
and what the reference computed from them:

- silu.pt        vllm_rlt.kernels.activation.silu_and_mul_reference
- attention.pt   vllm_rlt.kernels.paged_attention.torch_paged_attention and
                 KVCacheManager.write/attend (mixed request/depth rows, irregular pages)
- greedy.pt      vllm_rlt.worker.speculative.greedy_accept, logits.argmax(-1)
- sampler.pt     vllm_rlt.worker.sampler.Sampler.probabilities,
                 vllm_rlt.worker.speculative.rejection_sample (accept decisions, residuals)
- rollback.pt    KVCacheManager.truncate_suffix validity frontiers, slot mapping
- async_accept.pt  the tensor program of AsyncSpeculativeRunner._accept_and_update_state
"""

from __future__ import annotations

from pathlib import Path

import torch

from vllm_rlt.core.kv_cache_manager import KVCacheManager
from vllm_rlt.kernels.activation import silu_and_mul_reference
from vllm_rlt.kernels.paged_attention import torch_paged_attention
from vllm_rlt.sampling_params import SamplingParams
from vllm_rlt.worker.sampler import Sampler
from vllm_rlt.worker.speculative import greedy_accept, rejection_sample

HERE = Path(__file__).resolve().parent
torch.set_num_threads(1)


def golden_silu():
    cases = []
    # Known values of the reference's own test (tests/test_activation.py:49-53).
    gate, up = torch.tensor([0.0, 1.0, -1.0]), torch.tensor([2.0, 3.0, 4.0])
    cases.append(dict(gate=gate, up=up, out=silu_and_mul_reference(gate, up),
                      known=torch.tensor([0.0, 2.1931758, -1.0757657])))
    g = torch.Generator().manual_seed(42)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for shape in ((7,), (2, 7), (3, 129), (5, 688)):
            gate = (torch.randn(shape, generator=g) * 3).to(dtype)
            up = torch.randn(shape, generator=g).to(dtype)
            cases.append(dict(gate=gate, up=up, out=silu_and_mul_reference(gate, up)))
        info = torch.finfo(dtype)
        values = torch.tensor([float("nan"), float("inf"), -float("inf"), -100, -12, -1, -0.0, 0.0,
                               1, 12, 100, info.tiny, info.max], dtype=dtype)
        gate, up = torch.meshgrid(values, values, indexing="ij")
        gate, up = gate.contiguous(), up.contiguous()
        cases.append(dict(gate=gate, up=up, out=silu_and_mul_reference(gate, up), special=True))
    torch.save(cases, HERE / "silu.pt")


def golden_attention():
    cases = []
    # (a) direct torch_paged_attention over a permuted pool, zero-length row, GQA ratios.
    for seed, dtype, heads, kv_heads, head_dim, block, lengths in (
        (1, torch.float32, 8, 4, 64, 16, [0, 1, 15, 16, 17, 100]),
        (2, torch.bfloat16, 4, 4, 128, 16, [33, 5, 64, 129]),
        (3, torch.float16, 6, 2, 32, 4, [7, 9, 1]),
        (4, torch.float32, 4, 2, 7, 2, [5, 3, 6]),
        (5, torch.bfloat16, 4, 4, 128, 16, [100, 101, 102, 103, 104]),
    ):
        g = torch.Generator().manual_seed(seed)
        pages = (max(-(-n // block) for n in lengths) if seed == 5 else sum(-(-n // block) for n in lengths)) + 3
        k = (torch.randn(pages, block, kv_heads, head_dim, generator=g)).to(dtype)
        v = (torch.randn(pages, block, kv_heads, head_dim, generator=g)).to(dtype)
        order = torch.randperm(pages, generator=g).tolist()
        width = max(-(-n // block) for n in lengths)
        tables = torch.full((len(lengths), width), -1, dtype=torch.int32)
        if seed == 5:  # the k+1 rows of one request share one table
            ids = [order.pop() for _ in range(width)]
            for row in range(len(lengths)):
                tables[row] = torch.tensor(ids, dtype=torch.int32)
        else:
            for row, n in enumerate(lengths):
                ids = [order.pop() for _ in range(-(-n // block))]
                tables[row, : len(ids)] = torch.tensor(ids, dtype=torch.int32)
        q = torch.randn(len(lengths), heads, head_dim, generator=g).to(dtype)
        context = torch.tensor(lengths, dtype=torch.int32)
        safe = tables.clamp_min(0)  # the reference indexes with the padded table directly
        out = torch_paged_attention(q, k, v, safe, context)
        cases.append(dict(kind="direct", q=q, k=k, v=v, tables=tables, lengths=context, out=out))
    # (b) through KVCacheManager: layer-strided cache views, depth planes, freed hole
    # (tests/test_attention.py:30-55 of the reference).
    for head_dim in (7, 32):
        torch.manual_seed(48)
        cache = KVCacheManager(2, 2, head_dim, 48, 3, 3)
        cache.allocate("retained", 4)
        cache.allocate("hole", 8)
        cache.allocate("a", 7)
        cache.free("hole")
        cache.allocate("b", 6)
        for request_id, length in [("a", 7), ("b", 6)]:
            for depth in range(3):
                k = torch.randn(length, 2, head_dim) + depth * 0.5
                v = torch.randn_like(k) + (4 if request_id == "a" else -4)
                cache.write(1, [request_id] * length, [depth] * length, list(range(length)), k, v)
        request_ids, depths, positions = ["a", "b", "a", "b"], [2, 0, 1, 2], [6, 4, 2, 5]
        q = torch.randn(4, 6, head_dim)
        out = cache.attend(1, request_ids, depths, positions, q)
        batch = cache._prepare_batch(request_ids, depths, positions, for_write=False)
        cases.append(dict(kind="manager", q=q, key_cache=cache.key_cache.clone(),
                          value_cache=cache.value_cache.clone(), layer=1,
                          tables=batch.block_tables.clone(), lengths=batch.context_lengths.clone(),
                          out=out))
    torch.save(cases, HERE / "attention.pt")


def golden_greedy():
    table = []
    for k in (0, 1, 2, 4, 8):  # tests/test_speculative.py:225-233 of the reference
        candidates = list(range(100, 100 + k))
        for rejected in range(k + 1):
            targets = candidates[:rejected] + [7] + list(range(200, 200 + k - rejected))
            tokens, accepted = greedy_accept(candidates, targets)
            table.append(dict(candidates=candidates, targets=targets, tokens=tokens, accepted=accepted))
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(12, 1024, generator=g) * 3
    logits[3, 100] = logits[3, 900] = 50.0  # tie: lowest index wins
    logits[5] = 0.0
    argmax = dict(logits=logits, targets=logits.argmax(-1),
                  bf16_logits=logits.bfloat16(), bf16_targets=logits.bfloat16().argmax(-1))
    torch.save(dict(table=table, argmax=argmax), HERE / "greedy.pt")


def golden_async_accept():
    """AsyncSpeculativeRunner._accept_and_update_state (worker/async_speculative.py:417-447)
    re-run as the same tensor program on CPU for seeded ragged rounds."""
    g = torch.Generator().manual_seed(11)
    n, width = 9, 5
    counts = torch.randint(1, width + 1, (n,), generator=g)
    rows = int(counts.sum())
    request_rows = torch.repeat_interleave(torch.arange(n), counts)
    row_offsets = torch.cat([torch.arange(int(c)) for c in counts])
    starts = torch.randint(3, 500, (n,), generator=g)
    target = torch.randint(0, 50, (rows,), generator=g)
    tokens = torch.randint(0, 50, (n, width), generator=g)
    for i in range(n):  # make a prefix of the drafts agree with the targets
        agree = int(torch.randint(0, int(counts[i]), (1,), generator=g))
        first = int((request_rows == i).nonzero()[0])
        tokens[i, 1 : 1 + agree] = target[first : first + agree]
    drafts_count = counts - 1
    targets = torch.zeros((n, width), dtype=torch.long)
    targets[request_rows, row_offsets] = target
    drafts = torch.arange(width - 1)[None, :] < drafts_count[:, None]
    matches = (tokens[:, 1:] == targets[:, :-1]) & drafts
    accepted = matches.long().cumprod(1).sum(1)
    next_tokens = targets.gather(1, accepted[:, None]).squeeze(1)
    next_positions = starts + accepted + 1
    slots = torch.randperm(2 * n, generator=g)[:n]
    slot_values = torch.full((2 * n, 2), -7, dtype=torch.long)
    slot_values[slots] = torch.stack((next_tokens, next_positions), 1)
    result = torch.cat([target, accepted, next_positions])
    torch.save(dict(counts=counts, starts=starts, target=target, tokens=tokens, slots=slots,
                    slot_values=slot_values, result=result), HERE / "async_accept.pt")


def golden_sampler():
    out = dict(probabilities=[], rejection=[], distribution=[], filtered=[])
    g = torch.Generator().manual_seed(5)
    for vocab, temperature, scale in ((4, 1.0, 1.0), (64, 0.7, 1.0), (1024, 0.8, 3.0), (4099, 1.3, 3.0)):
        logits = torch.randn(vocab, generator=g) * scale
        probs = Sampler.probabilities(logits, SamplingParams(temperature=temperature))
        out["probabilities"].append(dict(logits=logits, temperature=temperature, probs=probs))
    logits = torch.tensor([0.50, 0.25, 0.15, 0.10]).log()  # tests/test_speculative.py:423-425
    out["probabilities"].append(dict(logits=logits, temperature=1.0,
                                     probs=Sampler.probabilities(logits, SamplingParams(temperature=1))))
    # rejection_sample decisions with the uniform it drew (same generator state replayed).
    for case in range(64):
        vocab = 1024
        target_logits = torch.randn(vocab, generator=g) * 3
        noise = (0.0, 0.5, 3.0)[case % 3]
        draft_logits = target_logits + torch.randn(vocab, generator=g) * noise
        if case % 3 == 2:
            draft_logits = torch.randn(vocab, generator=g) * 3
        params = SamplingParams(temperature=0.8)
        p = Sampler.probabilities(target_logits, params)
        q = Sampler.probabilities(draft_logits, params)
        candidate = int(torch.multinomial(q, 1, generator=g))
        replay = torch.Generator().set_state(g.get_state())
        uniform = float(torch.rand((), generator=replay))
        token, accepted = rejection_sample(candidate, p, q, g)
        residual = (p - q).clamp_min(0)
        out["rejection"].append(dict(target_logits=target_logits, draft_logits=draft_logits,
                                     temperature=0.8, candidate=candidate, uniform=uniform,
                                     accepted=bool(accepted), token=int(token),
                                     p_c=float(p[candidate]), q_c=float(q[candidate]),
                                     residual=residual / residual.sum()))
    # p/q pairs of tests/test_speculative.py:396-420 (distribution recovery).
    for p, q in (([0.1, 0.6, 0.3], [0.7, 0.2, 0.1]), ([0.0, 1.0, 0.0], [1.0, 0.0, 0.0]),
                 ([0.2, 0.3, 0.5], [0.2, 0.3, 0.5])):
        out["distribution"].append(dict(p=torch.tensor(p), q=torch.tensor(q)))
    # top-k / top-p supports and distributions (Sampler.probabilities, worker/sampler.py:40-54), drawn
    # after everything above so the earlier cases keep their generator stream.
    def filtered(logits, temperature, top_k, top_p, tied=False):
        params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p)
        out["filtered"].append(dict(logits=logits, temperature=temperature, top_k=top_k, top_p=top_p, tied=tied,
                                    probs=Sampler.probabilities(logits, params)))
    # the reference's own cases: tests/test_sampler.py:87-166, tests/test_speculative.py:423-434
    filtered(torch.tensor([5.0, 4.0, 4.0, 1.0]), 1.0, 2, 1.0, tied=True)
    filtered(torch.zeros(4), 1.0, 1, 1.0, tied=True)
    filtered(torch.tensor([1.0, 2.0, 3.0]), 1.0, 3, 1.0)
    filtered(torch.tensor([1.0, 2.0, 3.0]), 1.0, 5, 1.0)
    filtered(torch.tensor([4.0, 3.0, 2.0, 1.0]), 1.0, 3, 0.8)
    filtered(torch.linspace(1.0, 0.0, 100), 1.0, -1, 0.005)
    filtered(torch.tensor([1.0, 0.9, 0.8, 0.7]), 1.0, -1, 0.5)
    filtered(torch.tensor([0.50, 0.25, 0.15, 0.10]).log(), 1.0, -1, 0.8)
    filtered(torch.tensor([0.50, 0.25, 0.15, 0.10]).log(), 0.5, 2, 1.0)
    for vocab, temperature, scale, top_k, top_p in (
            (64, 0.7, 1.0, 8, 1.0), (64, 0.7, 1.0, -1, 0.9), (64, 1.0, 2.0, 16, 0.5),
            (1024, 0.8, 3.0, 50, 1.0), (1024, 0.8, 3.0, -1, 0.95), (1024, 0.8, 3.0, 40, 0.9),
            (1024, 1.5, 1.0, -1, 0.3), (1024, 1.5, 1.0, 1000, 0.999), (1024, 0.3, 3.0, 5, 0.99),
            (4099, 1.3, 3.0, 257, 0.9), (4099, 0.8, 3.0, -1, 0.8), (4099, 2.0, 0.5, 4098, 0.6),
            (4099, 1.0, 3.0, 1, 0.5), (4099, 1.0, 3.0, -1, 0.01)):
        filtered(torch.randn(vocab, generator=g) * scale, temperature, top_k, top_p)
    torch.save(out, HERE / "sampler.pt")


def golden_rollback():
    """truncate_suffix frontiers (tests/test_speculative.py:251-266 of the reference) and the
    next-round slot mapping write_block = table[plane][pos // B], write_offset = pos % B."""
    cases = []
    for block, start, count, emitted in ((2, 3, 4, 2), (16, 30, 5, 1), (16, 47, 5, 5), (4, 9, 3, 3)):
        planes, layers = 4, 2
        cache = KVCacheManager(layers, 2, 8, 256, block, planes)
        cache.allocate("r", start + count + 1)
        kv = torch.randn(start + count, 2, 8)
        for d in range(planes):
            for layer in range(layers):
                cache.write(layer, ["r"] * (start + count), [d] * (start + count),
                            list(range(start + count)), kv, kv)
        allocation = cache._get_allocation("r")
        before = [[w.prefix for w in plane] for plane in allocation.written]
        frontier = start + emitted
        cache.truncate_suffix("r", frontier)
        after = [[w.prefix for w in plane] for plane in allocation.written]
        tables = torch.tensor(allocation.block_tables, dtype=torch.int32)
        cases.append(dict(block=block, start=start, emitted=emitted, frontier=frontier,
                          tables=tables, before=torch.tensor(before), after=torch.tensor(after),
                          write_blocks=tables[:, frontier // block].long(),
                          write_offset=frontier % block, context_length=frontier + 1))
    # shared-prefix refusal: a page referenced by two requests must not be truncated.
    cache = KVCacheManager(1, 1, 4, 64, 2, 2, enable_prefix_caching=False)
    cache.allocate("a", 8)
    allocation = cache._get_allocation("a")
    page = allocation.block_tables[0][2]
    cache._refs[page] += 1
    try:
        cache.truncate_suffix("a", 3)
        refused = False
    except ValueError:
        refused = True
    cache.truncate_suffix("a", 6)  # pages at/after 6 // 2 = 3 are private: allowed
    refcounts = torch.tensor([cache._refs[b] for b in range(64)], dtype=torch.int32)
    cases.append(dict(shared=True, refused=refused, block=2,
                      tables=torch.tensor(allocation.block_tables, dtype=torch.int32),
                      refcounts=refcounts, refused_frontier=3, allowed_frontier=6))
    torch.save(cases, HERE / "rollback.pt")


if __name__ == "__main__":
    golden_silu()
    golden_attention()
    golden_greedy()
    golden_async_accept()
    golden_sampler()
    golden_rollback()
    for path in sorted(HERE.glob("*.pt")):
        print(path.name, path.stat().st_size)
