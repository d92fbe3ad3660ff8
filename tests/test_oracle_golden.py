"""Pins the CPU oracle (oracle/rlt_oracle.c) against vectors produced by the vllm-rlt
reference itself (tests/golden/make_golden.py) and against the known-answer values of the
reference's own tests.  Runs without a GPU."""

import pytest
import torch

from oracle import oracle


def _bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


def test_silu_known_values_and_reference_outputs(golden):
    cases = golden("silu.pt")
    known = cases[0]
    torch.testing.assert_close(oracle.silu_and_mul(known["gate"], known["up"]), known["known"])
    for case in cases:
        got = oracle.silu_and_mul(case["gate"], case["up"])
        want = case["out"]
        assert got.shape == want.shape and got.dtype == want.dtype
        if want.dtype == torch.float32:
            # libm expf vs torch's vectorised exp differ by an ulp or two in fp32.
            torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-30, equal_nan=True)
        else:
            # 16-bit outputs: identical except where that last fp32 ulp crosses a rounding
            # boundary of the activation (then one unit in the last place of the product).
            nan = torch.isnan(want)
            assert torch.equal(torch.isnan(got), nan)
            diff = (_bits(got)[~nan].int() - _bits(want)[~nan].int()).abs()
            assert int(diff.max()) <= 1
            assert float((diff != 0).float().mean()) < 2e-3


def test_silu_staged_fp64_contract():
    # The contract the reference states in tests/test_activation.py:56-75: round the
    # activation to the storage type, then round the product once.
    g = torch.Generator().manual_seed(42)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        gate = torch.randn(2, 3, 9, generator=g).to(dtype)
        up = torch.randn(2, 3, 9, generator=g).to(dtype)
        activated = (gate.double() * torch.sigmoid(gate.double())).to(dtype)
        expected = (activated.double() * up.double()).to(dtype)
        torch.testing.assert_close(oracle.silu_and_mul(gate, up), expected)


def test_attention_matches_reference_outputs(golden):
    for case in golden("attention.pt"):
        if case["kind"] == "direct":
            k, v = case["k"], case["v"]
        else:
            k, v = case["key_cache"][:, case["layer"]], case["value_cache"][:, case["layer"]]
        got = oracle.paged_attention(case["q"], k, v, case["tables"], case["lengths"])
        tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 2e-2}[case["q"].dtype]
        torch.testing.assert_close(got, case["out"], rtol=tol, atol=tol)
        zero_rows = (case["lengths"] == 0).nonzero().flatten().tolist()
        for row in zero_rows:
            assert torch.count_nonzero(got[row]) == 0


def test_windowed_attention_matches_reference_outputs(golden):
    data = golden("windowed.pt")
    for case in data["grid"]:
        for (window, length), want in case["out"].items():
            got = oracle.paged_attention_windowed(case["q"], case["key"], case["value"], case["tables"],
                                                  torch.tensor([length], dtype=torch.int32), window)
            torch.testing.assert_close(got, want, atol=2e-6, rtol=2e-5)     # the reference's own bounds for its Triton kernel
    case = data["batched"]
    for window, want in case["out"].items():
        got = oracle.paged_attention_windowed(case["q"], case["key"], case["value"], case["tables"], case["lengths"], window)
        torch.testing.assert_close(got.float(), want.float(), atol=8e-3, rtol=8e-3)   # one bf16 rounding of the output


def test_attention_packed_rows_equal_per_row_expansion():
    g = torch.Generator().manual_seed(3)
    block, heads, dim = 4, 2, 16
    k = torch.randn(12, block, heads, dim, generator=g)
    v = torch.randn(12, block, heads, dim, generator=g)
    tables = torch.tensor([[3, 7, 1, 0], [5, 2, 9, 11]], dtype=torch.int32)
    lengths = torch.tensor([9, 14], dtype=torch.int32)
    cu = torch.tensor([0, 3, 8], dtype=torch.int32)
    q = torch.randn(8, heads, dim, generator=g)
    packed = oracle.paged_attention(q, k, v, tables, lengths, cu)
    row_tables = torch.stack([tables[0]] * 3 + [tables[1]] * 5)
    row_lengths = torch.tensor([7, 8, 9, 10, 11, 12, 13, 14], dtype=torch.int32)
    rows = oracle.paged_attention(q, k, v, row_tables, row_lengths)
    assert torch.equal(packed, rows)


def test_greedy_accept_table_and_argmax(golden):
    data = golden("greedy.pt")
    for row in data["table"]:
        candidates, targets = row["candidates"], row["targets"]
        vocab = 300
        logits = torch.full((len(targets), vocab), -100.0)
        for j, t in enumerate(targets):
            logits[j, t] = 100.0
        tokens = torch.tensor([[5] + candidates], dtype=torch.int64)
        cu = torch.tensor([0, len(targets)], dtype=torch.int32)
        starts = torch.tensor([40], dtype=torch.int64)
        result = oracle.accept_greedy(logits, cu, tokens, starts)
        rows = len(targets)
        accepted = int(result[rows])
        assert accepted == row["accepted"]
        assert result[:rows].tolist() == targets
        assert result[: accepted + 1].tolist() == row["tokens"]
        assert int(result[rows + 1]) == 40 + accepted + 1
    arg = data["argmax"]
    assert torch.equal(oracle.argmax_rows(arg["logits"]), arg["targets"])
    assert torch.equal(oracle.argmax_rows(arg["bf16_logits"]), arg["bf16_targets"])
    assert int(oracle.argmax_rows(arg["logits"])[3]) == 100  # tie -> lowest index


def test_argmax_nan_counts_as_maximum():
    logits = torch.tensor([[1.0, float("nan"), 5.0, float("nan")], [float("-inf")] * 4])
    assert oracle.argmax_rows(logits).tolist() == logits.argmax(-1).tolist() == [1, 0]


def test_async_accept_program(golden):
    data = golden("async_accept.pt")
    counts = data["counts"]
    n, rows = counts.numel(), int(counts.sum())
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    vocab = 64
    logits = torch.full((rows, vocab), -50.0)
    logits[torch.arange(rows), data["target"]] = 50.0
    slot_values = torch.full_like(data["slot_values"], -7)
    result = oracle.accept_greedy(logits, cu, data["tokens"], data["starts"], data["slots"],
                                  slot_values)
    assert torch.equal(result, data["result"])
    assert torch.equal(slot_values, data["slot_values"])


def test_probabilities_match_reference_sampler(golden):
    data = golden("sampler.pt")
    for case in data["probabilities"]:
        probs, status = oracle.probabilities(case["logits"], case["temperature"])
        assert status == 0
        torch.testing.assert_close(probs, case["probs"], rtol=2e-6, atol=1e-12)
        assert abs(float(probs.double().sum()) - 1.0) < 1e-5


def test_top_k_top_p_supports_and_distributions_match_reference_sampler(golden):
    """Sampler.probabilities with filters: the support (which tokens stay) is exact, the
    probabilities agree to fp32 rounding.  Among tied logits the reference leaves the
    survivor unspecified (tests/test_sampler.py:101-103); the canonical order keeps the lower
    index, so tied cases compare the sorted values."""
    cases = golden("sampler.pt")["filtered"]
    assert len(cases) >= 20
    for case in cases:
        probs, status = oracle.probabilities(case["logits"], case["temperature"], case["top_k"], case["top_p"])
        assert status == 0
        if case["tied"]:
            torch.testing.assert_close(probs.sort().values, case["probs"].sort().values, rtol=2e-6, atol=1e-12)
            support = probs.nonzero().flatten().tolist()
            assert support == sorted(support)[:len(support)] and support[0] == 0
        else:
            assert torch.equal(probs > 0, case["probs"] > 0), (case["top_k"], case["top_p"])
            torch.testing.assert_close(probs, case["probs"], rtol=4e-6, atol=1e-12)
        assert abs(float(probs.double().sum()) - 1.0) < 1e-5


def test_top_k_ties_keep_the_lowest_indices_and_top_p_cuts_inside_a_tie_group():
    # canonical tie order: (logit descending, index ascending)
    probs, _ = oracle.probabilities(torch.tensor([5.0, 4.0, 4.0, 1.0]), 1.0, 2, 1.0)
    assert probs.nonzero().flatten().tolist() == [0, 1]
    probs, _ = oracle.probabilities(torch.zeros(8), 1.0, 3, 1.0)
    assert probs.nonzero().flatten().tolist() == [0, 1, 2]
    # eight tied tokens of mass 1/8: the ranks whose preceding mass is <= 0.3 are 0, 1, 2
    probs, _ = oracle.probabilities(torch.zeros(8), 1.0, -1, 0.3)
    assert probs.nonzero().flatten().tolist() == [0, 1, 2]
    torch.testing.assert_close(probs[:3], torch.full((3,), 1 / 3))
    # top-k first, then top-p over the top-k distribution
    probs, _ = oracle.probabilities(torch.tensor([0.0, 1.0, 1.0, 1.0, 1.0, -1.0]), 1.0, 3, 0.5)
    assert probs.nonzero().flatten().tolist() == [1, 2]


def test_filtered_sampling_never_leaves_the_support():
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(32, 777, generator=g) * 2
    temperature = torch.full((32,), 0.9)
    top_k = torch.randint(1, 40, (32,), generator=g, dtype=torch.int32)
    top_p = torch.rand(32, generator=g) * 0.9 + 0.05
    tokens, status = oracle.sample_rows(logits, temperature, torch.rand(32, generator=g), top_k, top_p)
    assert not status.any()
    for r in range(32):
        probs, _ = oracle.probabilities(logits[r], 0.9, int(top_k[r]), float(top_p[r]))
        assert probs[tokens[r]] > 0 and int((probs > 0).sum()) <= int(top_k[r])


def test_rejection_decisions_match_reference(golden):
    data = golden("sampler.pt")
    accepted_count = 0
    for case in data["rejection"]:
        vocab = case["target_logits"].numel()
        target = torch.stack([case["target_logits"], torch.zeros(vocab)])
        draft = torch.stack([case["draft_logits"], torch.zeros(vocab)])
        tokens = torch.tensor([[0, case["candidate"]]], dtype=torch.int64)
        cu = torch.tensor([0, 2], dtype=torch.int32)
        starts = torch.tensor([10], dtype=torch.int64)
        temperature = torch.tensor([case["temperature"]])
        u_accept = torch.tensor([case["uniform"], 0.0])
        # The decision must agree with the reference unless u*q is within rounding of p.
        margin = abs(case["uniform"] * case["q_c"] - case["p_c"]) / max(case["p_c"], 1e-30)
        for u_final in (0.0, 0.37, 0.999):
            result, status = oracle.accept_rejection(target, draft, cu, tokens, starts, temperature,
                                                     u_accept, torch.tensor([u_final]))
            assert int(status[0]) == 0
            accepted = int(result[2])
            if margin > 1e-4:
                assert accepted == int(case["accepted"])
            if accepted:
                assert int(result[0]) == case["candidate"]
            else:
                # A residual draw can only return a token with residual mass.
                assert float(case["residual"][int(result[0])]) > 0
            assert int(result[3]) == 10 + accepted + 1
        accepted_count += int(case["accepted"])
    assert 0 < accepted_count < len(data["rejection"])


def test_residual_draw_follows_the_reference_residual_distribution(golden):
    # Inverse CDF over a fine grid of uniforms reproduces max(p - q, 0) / sum.
    case = next(c for c in golden("sampler.pt")["rejection"] if not c["accepted"])
    vocab = case["target_logits"].numel()
    target = torch.stack([case["target_logits"], torch.zeros(vocab)])
    draft = torch.stack([case["draft_logits"], torch.zeros(vocab)])
    tokens = torch.tensor([[0, case["candidate"]]], dtype=torch.int64)
    cu = torch.tensor([0, 2], dtype=torch.int32)
    counts = torch.zeros(vocab)
    draws = 4000
    for i in range(draws):
        result, _ = oracle.accept_rejection(target, draft, cu, tokens, torch.tensor([0]),
                                            torch.tensor([case["temperature"]]),
                                            torch.tensor([case["uniform"], 0.0]),
                                            torch.tensor([(i + 0.5) / draws]))
        counts[int(result[0])] += 1
    torch.testing.assert_close(counts / draws, case["residual"], atol=2.0 / draws, rtol=0)


@pytest.mark.parametrize("index", [0, 1, 2])
def test_rejection_sampling_recovers_target_distribution(golden, index):
    # The statistical contract of tests/test_speculative.py:396-420 of the reference, with the
    # generator replaced by seeded uniforms fed through the oracle's explicit-uniform interface.
    case = golden("sampler.pt")["distribution"][index]
    p, q = case["p"], case["q"]
    logits_p = torch.where(p > 0, p.log(), torch.tensor(-80.0))
    logits_q = torch.where(q > 0, q.log(), torch.tensor(-80.0))
    g = torch.Generator().manual_seed(431)
    n = 12000
    uniforms = torch.rand(n, 3, generator=g)
    temperature = torch.ones(n)
    candidates, status = oracle.sample_rows(logits_q.expand(n, 3).contiguous(), temperature,
                                            uniforms[:, 0].contiguous())
    assert int(status.abs().sum()) == 0
    target = torch.stack([logits_p, logits_p]).repeat(n, 1)
    draft = torch.stack([logits_q, logits_q]).repeat(n, 1)
    tokens = torch.stack([torch.zeros(n, dtype=torch.int64), candidates], 1)
    cu = (torch.arange(n + 1) * 2).int()
    u_accept = torch.stack([uniforms[:, 1], torch.zeros(n)], 1).flatten().contiguous()
    result, status = oracle.accept_rejection(target, draft, cu, tokens,
                                             torch.zeros(n, dtype=torch.int64), temperature,
                                             u_accept, uniforms[:, 2].contiguous())
    assert int(status.abs().sum()) == 0
    first = result[: 2 * n].view(n, 2)[:, 0]
    counts = torch.bincount(first, minlength=3).float()
    torch.testing.assert_close(counts / counts.sum(), p, atol=0.016, rtol=0)


def test_zero_proposal_and_bad_logits_are_reported():
    vocab = 8
    target = torch.zeros(2, vocab)
    draft = torch.zeros(2, vocab)
    draft[0, 3] = -2000.0  # q[3] underflows to exactly zero
    tokens = torch.tensor([[0, 3]], dtype=torch.int64)
    cu = torch.tensor([0, 2], dtype=torch.int32)
    args = (cu, tokens, torch.tensor([5]), torch.tensor([1.0]), torch.tensor([0.5, 0.0]),
            torch.tensor([0.5]))
    _, status = oracle.accept_rejection(target, draft, *args)
    assert int(status[0]) == 1
    target[0, 0] = float("nan")
    draft[0, 3] = 0.0
    _, status = oracle.accept_rejection(target, draft, *args)
    assert int(status[0]) == 3


def test_rollback_frontiers_and_slot_mapping(golden):
    for case in golden("rollback.pt"):
        if case.get("shared"):
            tables = case["tables"][None]
            for frontier, want in ((case["refused_frontier"], 4), (case["allowed_frontier"], 0)):
                out = oracle.rollback(torch.tensor([0]), torch.tensor([frontier]), tables,
                                      case["block"], refcounts=case["refcounts"])
                assert int(out[4][0]) == want
            assert case["refused"]
            continue
        tables = case["tables"][None].contiguous()
        prefix = case["before"][None].clone().long()
        frontier, lengths, blocks, offsets, status = oracle.rollback(
            torch.tensor([case["start"]]), torch.tensor([case["emitted"]]), tables, case["block"],
            written_prefix=prefix)
        assert int(status[0]) == 0
        assert int(frontier[0]) == case["frontier"]
        assert torch.equal(prefix[0], case["after"].long())
        assert int(lengths[0]) == case["context_length"]
        assert int(offsets[0]) == case["write_offset"]
        assert torch.equal(blocks[0], case["write_blocks"])


def test_finalize_tokens_match_the_reference_pools(golden):
    for case in golden("finalize.pt"):
        key, value = case["key_before"].clone(), case["value_before"].clone()
        oracle.finalize_tokens(key, value, case["tables"], case["slots"], case["depths"], case["positions"])
        assert torch.equal(key.view(torch.uint8), case["key_after"].view(torch.uint8))
        assert torch.equal(value.view(torch.uint8), case["value_after"].view(torch.uint8))
        assert not torch.equal(case["key_before"], case["key_after"])


def _pipeline_inputs(step, n):
    widths = step["widths"]
    row_starts = torch.zeros(n, dtype=torch.int32)
    row_starts[1:] = widths.cumsum(0)[:-1].int()
    return widths, row_starts


def test_pipeline_shift_matches_every_reference_step(golden):
    data = golden("pipeline.pt")
    seen = set()
    for step in data["steps"]:
        before, after = step["before"], step["after"]
        n = before["tokens"].shape[0]
        state = {k: before[k].clone() for k in ("tokens", "depths", "candidates", "hidden", "token", "position")}
        state["active"] = before["active"].to(torch.uint8)
        widths, row_starts = _pipeline_inputs(step, n)
        result = oracle.pipeline_shift(state, widths, row_starts, step["choices"], step["step_hidden"],
                                       data["limits"], data["draft_loops"], data["target_loops"])
        assert torch.equal(result, after["result"])
        for key in ("tokens", "depths", "candidates", "token", "position"):
            assert torch.equal(state[key], after[key]), key
        assert torch.equal(state["active"].bool(), after["active"])
        assert torch.equal(state["hidden"], after["hidden"])
        for row in after["result"].view(n, 6).tolist():
            seen.add((row[1], row[2]))
    assert seen == {(0, 0), (0, 1), (1, 1)}  # waiting, rejected and accepted steps all occur


def test_rope_and_sandwich_norm_match_the_reference_layers(golden):
    """apply_rotary_pos_emb is reproduced bit for bit; RMSNorm and the sandwich residual flow to
    the last place of the dtype (the reference's fp32 mean has no specified summation order)."""
    data = golden("layers.pt")
    for case in data["rope"]:
        q, k = case["q"], case["k"]
        rows, kv_heads, dim = k.shape
        key_cache = torch.zeros(rows, 1, kv_heads, dim, dtype=q.dtype)
        value_cache = torch.zeros_like(key_cache)
        blocks, offsets = torch.arange(rows), torch.zeros(rows, dtype=torch.int64)
        q_rot = oracle.rope_kv_write(q, k, k, case["cos"], case["sin"], key_cache, value_cache, blocks, offsets)
        assert torch.equal(q_rot, case["q_rot"]) and torch.equal(key_cache[:, 0], case["k_rot"])
        assert torch.equal(value_cache[:, 0], k)
    ulp = {torch.float32: 2.0 ** -23, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}
    for case in data["norm"]:
        dtype = case["x"].dtype
        plain, _ = oracle.sandwich_norm(case["x"], case["weight"], case["eps"])
        total, following = oracle.sandwich_norm(case["x"], case["weight"], case["eps"], case["residual"], case["weight2"])
        for got, want in ((plain, case["plain"]), (total, case["total"])):
            # the residual add cancels, so the last place is that of the operands, not of the sum
            torch.testing.assert_close(got.float(), want.float(), rtol=2 * ulp[dtype],
                                       atol=2 * ulp[dtype] * float(want.abs().max()))
            if dtype != torch.float32:   # a last-place difference of the fp32 scale rarely survives the rounding
                assert float((got == want).float().mean()) > 0.99
        torch.testing.assert_close(following.float(), case["following"].float(), rtol=4 * ulp[dtype],
                                   atol=4 * ulp[dtype] * float(case["following"].abs().max()))


def test_packed_prefill_matches_the_reference_rows(golden):
    case = golden("prefill.pt")
    out = oracle.paged_attention(case["q"], case["key"], case["value"], case["tables"].clamp_min(0), case["lengths"],
                                 case["cu_seqlens_q"])
    torch.testing.assert_close(out.float(), case["out"].float(), rtol=2e-2, atol=2e-2)
    assert float((out == case["out"]).float().mean()) > 0.95   # both round an fp32 result to bf16 once


def test_philox_known_answers_and_round_uniform_streams():
    # the published known-answer vectors of Philox4x32-10 (Random123 kat_vectors)
    assert oracle.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert oracle.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    seeds, rounds = torch.tensor([5, 5, 6]), torch.tensor([0, 1, 0])
    draft, accept, final = oracle.round_uniforms(seeds, rounds, 64)
    everything = torch.cat([draft.reshape(-1), accept.reshape(-1), final])
    assert float(everything.min()) >= 0.0 and float(everything.max()) < 1.0
    assert everything.unique().numel() > 0.99 * everything.numel()          # streams do not repeat each other
    assert abs(float(everything.mean()) - 0.5) < 0.05
    again = oracle.round_uniforms(seeds[:1], rounds[:1], 64)
    assert torch.equal(again[0][0], draft[0]) and torch.equal(again[1][0], accept[0])


def test_padded_rounds_decide_like_compact_rounds():
    # a round of fixed shape (every request owns k + 1 rows, row_counts says how many are real) gives the
    # decisions of the reference's compact layout; requests without rows are left alone
    g = torch.Generator().manual_seed(3)
    n, width, vocab = 9, 4, 97
    counts = torch.tensor([0, 4, 1, 3, 0, 2, 4, 1, 3], dtype=torch.int32)
    cu_padded = (torch.arange(n + 1) * width).int()
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    keep = (torch.arange(width)[None, :] < counts[:, None]).reshape(-1)
    target = torch.randn(n * width, vocab, generator=g) * 3
    draft = target + torch.randn(n * width, vocab, generator=g)
    tokens = torch.randint(0, vocab, (n, width), generator=g)
    tokens[:, 1:] = torch.where(torch.rand(n, width - 1, generator=g) < 0.7, target.argmax(-1).view(n, width)[:, :-1],
                                tokens[:, 1:])
    starts = torch.randint(5, 500, (n,), generator=g)
    temperature = torch.tensor([0.8, 0.8, 0.0, 0.8, 0.0, 0.8, 0.8, 0.8, 0.0])
    u_accept, u_final = torch.rand(n * width, generator=g), torch.rand(n, generator=g)
    rows, total = n * width, int(cu[-1])
    live = counts > 0
    for greedy in (True, False):
        slots = torch.arange(n)
        padded_slots, compact_slots = torch.full((n, 2), -3), torch.full((n, 2), -3)
        if greedy:
            padded = oracle.accept_greedy(target, cu_padded, tokens, starts, slots, padded_slots, counts)
            compact = oracle.accept_greedy(target[keep], cu, tokens, starts, slots, compact_slots)
        else:
            padded, status = oracle.accept_rejection(target, draft, cu_padded, tokens, starts, temperature, u_accept,
                                                     u_final, slots, padded_slots, row_counts=counts)
            compact, _ = oracle.accept_rejection(target[keep], draft[keep], cu, tokens, starts, temperature,
                                                 u_accept[keep], u_final, slots, compact_slots)
            assert status.tolist() == [0] * n
        assert torch.equal(padded[:rows][keep], compact[:total]) and bool((padded[:rows][~keep] == -1).all())
        assert torch.equal(padded[rows:rows + n][live], compact[total:total + n][live])
        assert torch.equal(padded[rows + n:][live], compact[total + n:][live])
        assert torch.equal(padded[rows + n:][~live], starts[~live]) and bool((padded[rows:rows + n][~live] == 0).all())
        assert torch.equal(padded_slots[live], compact_slots[live]) and bool((padded_slots[~live] == -3).all())


def test_rollback_accepts_a_frontier_at_the_end_of_the_allocation():
    tables = torch.arange(8, dtype=torch.int32).view(1, 2, 4)
    frontier, lengths, blocks, offsets, status = oracle.rollback(torch.tensor([60]), torch.tensor([4]), tables, 16)
    assert status.tolist() == [0] and frontier.tolist() == [64] and lengths.tolist() == [65]
    assert blocks.tolist() == [[-1, -1]] and offsets.tolist() == [0]
    assert oracle.rollback(torch.tensor([60]), torch.tensor([5]), tables, 16)[4].tolist() == [5]
