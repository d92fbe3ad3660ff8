"""Acceptance kernels vs the CPU oracle (bit-exact) and the reference's golden vectors."""

import pytest
import torch

import vllm_rlt_b200 as rlt
from oracle import oracle

pytestmark = pytest.mark.gpu


def make_round(n, k_max, vocab, dtype, seed, agree=True):
    g = torch.Generator().manual_seed(seed)
    counts = torch.randint(1, k_max + 2, (n,), generator=g)
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    rows = int(cu[-1])
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(dtype)
    tokens = torch.randint(0, vocab, (n, k_max + 1), generator=g)
    if agree:
        targets = logits.argmax(-1)
        for i in range(n):
            a = int(torch.randint(0, int(counts[i]), (1,), generator=g))
            tokens[i, 1:1 + a] = targets[int(cu[i]):int(cu[i]) + a]
    starts = torch.randint(1, 3000, (n,), generator=g)
    slots = torch.randperm(2 * n, generator=g)[:n]
    return dict(cu=cu, rows=rows, logits=logits, tokens=tokens, starts=starts, slots=slots, counts=counts, g=g)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("vocab", [49152, 1024, 1027, 7])
def test_argmax_matches_torch_and_oracle(dtype, vocab):
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(33, vocab, generator=g) * 3).to(dtype)
    logits[1, vocab // 2] = logits[1, vocab - 1] = 60.0
    logits[2] = 0.0
    logits[3, 0] = -0.0
    logits[4, vocab - 1] = float("nan")
    logits[5, 3 % vocab] = float("nan")
    logits[5, 5 % vocab] = float("inf")
    got = rlt.argmax_rows(logits.cuda()).cpu()
    assert torch.equal(got, oracle.argmax_rows(logits))
    assert torch.equal(got, logits.argmax(-1))
    # a strided row view (row stride > vocab) is honoured
    wide = torch.zeros(33, vocab + 5, dtype=dtype)
    wide[:, :vocab] = logits
    assert torch.equal(rlt.argmax_rows(wide.cuda()[:, :vocab]).cpu(), got)


def test_greedy_accept_table_of_the_reference(golden):
    for row in golden("greedy.pt")["table"]:
        candidates, targets = row["candidates"], row["targets"]
        logits = torch.full((len(targets), 300), -100.0)
        for j, t in enumerate(targets):
            logits[j, t] = 100.0
        tokens = torch.tensor([[5] + candidates], dtype=torch.int64)
        cu = torch.tensor([0, len(targets)], dtype=torch.int32)
        result = rlt.accept_greedy(logits.cuda(), cu.cuda(), tokens.cuda(), torch.tensor([40]).cuda()).cpu()
        results, frontiers = rlt.decode_result(result.tolist(), cu.tolist())
        assert results[0].accepted_count == row["accepted"]
        assert results[0].token_ids == row["tokens"]
        assert frontiers == [40 + row["accepted"] + 1]


def test_async_accept_program_of_the_reference(golden):
    data = golden("async_accept.pt")
    counts = data["counts"]
    n, rows = counts.numel(), int(counts.sum())
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    logits = torch.full((rows, 64), -50.0)
    logits[torch.arange(rows), data["target"]] = 50.0
    slot_values = torch.full_like(data["slot_values"], -7).cuda()
    result = rlt.accept_greedy(logits.cuda(), cu.cuda(), data["tokens"].cuda(), data["starts"].cuda(),
                               data["slots"].cuda(), slot_values)
    assert torch.equal(result.cpu(), data["result"])
    assert torch.equal(slot_values.cpu(), data["slot_values"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_round_matches_oracle_at_vocab_49152(dtype):
    r = make_round(64, 4, 49152, dtype, seed=21)
    want_slots = torch.full((128, 2), -1, dtype=torch.int64)
    want = oracle.accept_greedy(r["logits"], r["cu"], r["tokens"], r["starts"], r["slots"], want_slots)
    got_slots = torch.full((128, 2), -1, dtype=torch.int64).cuda()
    got = rlt.accept_greedy(r["logits"].cuda(), r["cu"].cuda(), r["tokens"].cuda(), r["starts"].cuda(),
                            r["slots"].cuda(), got_slots)
    assert torch.equal(got.cpu(), want) and torch.equal(got_slots.cpu(), want_slots)
    accepted = want[r["rows"]:r["rows"] + 64]
    assert int(accepted.max()) > 0 and int(accepted.min()) == 0


@pytest.mark.parametrize("vocab,dtype", [(49152, torch.float32), (4099, torch.float32), (49152, torch.bfloat16)])
def test_sample_rows_matches_oracle_bit_for_bit(vocab, dtype):
    g = torch.Generator().manual_seed(8)
    rows = 24
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(dtype)
    temperature = torch.tensor([0.8, 1.0, 0.0, 1.7] * 6)
    uniforms = torch.rand(rows, generator=g)
    uniforms[0], uniforms[1] = 0.0, 0.99999994
    want_tokens, want_status = oracle.sample_rows(logits, temperature, uniforms)
    got_tokens, got_status = rlt.sample_rows(logits.cuda(), temperature.cuda(), uniforms.cuda())
    assert torch.equal(got_tokens.cpu(), want_tokens) and torch.equal(got_status.cpu(), want_status)
    assert int(want_status.abs().sum()) == 0


@pytest.mark.parametrize("noise,dtype", [(0.0, torch.float32), (0.5, torch.float32), (3.0, torch.float32),
                                         (0.5, torch.bfloat16)])
def test_rejection_round_matches_oracle_bit_for_bit(noise, dtype):
    # draft logits: identical (all accept), target + N(0, 0.5) (mixed), independent (mostly reject)
    n, k, vocab = 32, 4, 49152
    r = make_round(n, k, vocab, torch.float32, seed=33, agree=False)
    g = r["g"]
    target = r["logits"]
    draft = target + torch.randn(r["rows"], vocab, generator=g) * noise if noise < 3 else \
        torch.randn(r["rows"], vocab, generator=g) * 3
    target, draft = target.to(dtype), draft.to(dtype)
    temperature = torch.full((n,), 0.8)
    temperature[::7] = 0.0   # greedy requests mixed into the batch
    # candidates are drawn from q with the same explicit-uniform rule
    per_row_t = torch.repeat_interleave(temperature, r["counts"])
    drafts, _ = oracle.sample_rows(draft, per_row_t, torch.rand(r["rows"], generator=g))
    tokens = r["tokens"]
    for i in range(n):
        a, c = int(r["cu"][i]), int(r["counts"][i])
        tokens[i, 1:c] = drafts[a:a + c - 1]
    u_accept, u_final = torch.rand(r["rows"], generator=g), torch.rand(n, generator=g)
    want_slots = torch.full((2 * n, 2), -1, dtype=torch.int64)
    want, want_status = oracle.accept_rejection(target, draft, r["cu"], tokens, r["starts"], temperature,
                                                u_accept, u_final, r["slots"], want_slots)
    got_slots = torch.full((2 * n, 2), -1, dtype=torch.int64).cuda()
    got, got_status = rlt.accept_rejection(target.cuda(), draft.cuda(), r["cu"].cuda(), tokens.cuda(),
                                           r["starts"].cuda(), temperature.cuda(), u_accept.cuda(),
                                           u_final.cuda(), r["slots"].cuda(), got_slots)
    assert torch.equal(got_status.cpu(), want_status) and int(want_status.abs().sum()) == 0
    assert torch.equal(got.cpu(), want)
    assert torch.equal(got_slots.cpu(), want_slots)
    accepted = want[r["rows"]:r["rows"] + n]
    drafts_per_request = r["counts"] - 1
    if noise == 0.0:
        sampled = temperature != 0
        assert torch.equal(accepted[sampled], drafts_per_request[sampled])
    if noise == 3.0:
        assert int(accepted.sum()) < int(drafts_per_request.sum()) // 2


def _oracle_probabilities(logits, temperature, top_k, top_p):
    rows = []
    for r in range(logits.shape[0]):
        probs, status = oracle.probabilities(logits[r], float(temperature[r]), int(top_k[r]), float(top_p[r]))
        assert status == 0
        rows.append(probs)
    return torch.stack(rows)


def test_filtered_probabilities_of_the_reference(golden):
    """Sampler.probabilities with top-k / top-p: support exact, values to fp32 rounding."""
    for case in golden("sampler.pt")["filtered"]:
        probs, status = rlt.probabilities(case["logits"][None].cuda(), torch.tensor([case["temperature"]]).cuda(),
                                          torch.tensor([case["top_k"]], dtype=torch.int32).cuda(),
                                          torch.tensor([case["top_p"]]).cuda())
        assert int(status[0]) == 0
        probs = probs[0].cpu()
        if case["tied"]:
            torch.testing.assert_close(probs.sort().values, case["probs"].sort().values, rtol=2e-6, atol=1e-12)
        else:
            assert torch.equal(probs > 0, case["probs"] > 0), (case["top_k"], case["top_p"])
            torch.testing.assert_close(probs, case["probs"], rtol=4e-6, atol=1e-12)


@pytest.mark.parametrize("vocab,dtype,levels", [(49152, torch.float32, 0), (49152, torch.bfloat16, 0),
                                                (4099, torch.float32, 0), (1027, torch.float32, 9),
                                                (49152, torch.float32, 33), (300, torch.float16, 0)])
def test_filtered_probabilities_match_oracle_bit_for_bit(vocab, dtype, levels):
    """The radix-select cut equals the oracle's full sort: same support, same bits.  `levels`
    quantises the logits so that cuts fall inside large tie groups."""
    g = torch.Generator().manual_seed(vocab + levels)
    rows = 20
    logits = torch.randn(rows, vocab, generator=g) * 3
    if levels:
        logits = (logits * levels / 12).round() * (12 / levels)
    logits = logits.to(dtype)
    logits[3, : vocab // 2] = float("-inf")
    temperature = torch.tensor([0.8, 1.0, 0.3, 1.7, 5.0] * 4)
    top_k = torch.tensor([-1, 1, 2, 50, vocab - 1, vocab, 7, 1000, -1, 40] * 2, dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.999, 0.3, 1.0, 0.01, 0.6, 0.8,
                          1.0, 0.7, 1.0, 1.0, 0.2, 1.0, 0.99, 0.9999999, 1e-6, 0.5])
    want = _oracle_probabilities(logits, temperature, top_k, top_p)
    got, status = rlt.probabilities(logits.cuda(), temperature.cuda(), top_k.cuda(), top_p.cuda())
    assert not status.any()
    assert torch.equal(got.cpu(), want)
    # no filters at all: the unfiltered distribution, whichever way it is requested
    plain, _ = rlt.probabilities(logits.cuda(), temperature.cuda())
    off, _ = rlt.probabilities(logits.cuda(), temperature.cuda(), torch.full((rows,), -1, dtype=torch.int32).cuda(),
                               torch.ones(rows).cuda())
    assert torch.equal(plain, off)
    assert torch.equal(plain.cpu(), _oracle_probabilities(logits, temperature, [-1] * rows, [1.0] * rows))


def test_probabilities_reject_greedy_and_bad_rows():
    logits = torch.randn(3, 64)
    logits[2, 5] = float("nan")
    probs, status = rlt.probabilities(logits.cuda(), torch.tensor([0.0, 1.0, 1.0]).cuda())
    assert status.tolist() == [3, 0, 3]
    assert not probs[0].any() and not probs[2].any()


@pytest.mark.parametrize("vocab,dtype", [(49152, torch.float32), (4099, torch.bfloat16)])
def test_filtered_sample_rows_match_oracle_bit_for_bit(vocab, dtype):
    g = torch.Generator().manual_seed(18)
    rows = 24
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(dtype)
    temperature = torch.tensor([0.8, 1.0, 0.0, 1.7] * 6)
    top_k = torch.tensor([-1, 50, 3, 1] * 6, dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.3, 0.99] * 4)
    uniforms = torch.rand(rows, generator=g)
    uniforms[0], uniforms[1] = 0.0, 0.99999994
    want_tokens, want_status = oracle.sample_rows(logits, temperature, uniforms, top_k, top_p)
    got_tokens, got_status = rlt.sample_rows(logits.cuda(), temperature.cuda(), uniforms.cuda(), top_k.cuda(),
                                             top_p.cuda())
    assert torch.equal(got_tokens.cpu(), want_tokens) and torch.equal(got_status.cpu(), want_status)
    assert int(want_status.abs().sum()) == 0
    plain_tokens, _ = oracle.sample_rows(logits, temperature, uniforms)
    assert not torch.equal(plain_tokens, want_tokens)      # the filters change the draws


@pytest.mark.parametrize("noise,dtype", [(0.5, torch.float32), (3.0, torch.float32), (0.5, torch.bfloat16)])
def test_filtered_rejection_round_matches_oracle_bit_for_bit(noise, dtype):
    """Per-request top-k / top-p filter both p and q; drafts are drawn from the filtered q."""
    n, k, vocab = 24, 4, 49152
    r = make_round(n, k, vocab, torch.float32, seed=35, agree=False)
    g = r["g"]
    target = r["logits"]
    draft = target + torch.randn(r["rows"], vocab, generator=g) * noise if noise < 3 else \
        torch.randn(r["rows"], vocab, generator=g) * 3
    target, draft = target.to(dtype), draft.to(dtype)
    temperature = torch.full((n,), 0.8)
    temperature[::7] = 0.0
    top_k = torch.tensor([-1, 50, 8, 2000] * 6, dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 0.95] * 8)
    rep = lambda t: torch.repeat_interleave(t, r["counts"])
    drafts, _ = oracle.sample_rows(draft, rep(temperature), torch.rand(r["rows"], generator=g), rep(top_k),
                                   rep(top_p))
    tokens = r["tokens"]
    for i in range(n):
        a, c = int(r["cu"][i]), int(r["counts"][i])
        tokens[i, 1:c] = drafts[a:a + c - 1]
    u_accept, u_final = torch.rand(r["rows"], generator=g), torch.rand(n, generator=g)
    want_slots = torch.full((2 * n, 2), -1, dtype=torch.int64)
    want, want_status = oracle.accept_rejection(target, draft, r["cu"], tokens, r["starts"], temperature,
                                                u_accept, u_final, r["slots"], want_slots, top_k, top_p)
    got_slots = torch.full((2 * n, 2), -1, dtype=torch.int64).cuda()
    got, got_status = rlt.accept_rejection(target.cuda(), draft.cuda(), r["cu"].cuda(), tokens.cuda(),
                                           r["starts"].cuda(), temperature.cuda(), u_accept.cuda(),
                                           u_final.cuda(), r["slots"].cuda(), got_slots, top_k=top_k.cuda(),
                                           top_p=top_p.cuda())
    assert torch.equal(got_status.cpu(), want_status)
    assert torch.equal(got.cpu(), want)
    assert torch.equal(got_slots.cpu(), want_slots)
    # a draft outside the target's support has p = 0 and is rejected; one outside q's support
    # would be a zero-probability proposal: drafts drawn from the filtered q never are
    assert not (want_status == 1).any()
    unfiltered, _ = oracle.accept_rejection(target, draft, r["cu"], tokens, r["starts"], temperature, u_accept,
                                            u_final)
    assert not torch.equal(unfiltered, want)


def test_rejection_decisions_of_the_reference(golden):
    for case in golden("sampler.pt")["rejection"]:
        vocab = case["target_logits"].numel()
        target = torch.stack([case["target_logits"], torch.zeros(vocab)]).cuda()
        draft = torch.stack([case["draft_logits"], torch.zeros(vocab)]).cuda()
        tokens = torch.tensor([[0, case["candidate"]]], dtype=torch.int64).cuda()
        cu = torch.tensor([0, 2], dtype=torch.int32).cuda()
        result, status = rlt.accept_rejection(target, draft, cu, tokens, torch.tensor([10]).cuda(),
                                              torch.tensor([case["temperature"]]).cuda(),
                                              torch.tensor([case["uniform"], 0.0]).cuda(),
                                              torch.tensor([0.37]).cuda())
        result = result.cpu()
        margin = abs(case["uniform"] * case["q_c"] - case["p_c"]) / max(case["p_c"], 1e-30)
        assert int(status[0]) == 0
        if margin > 1e-4:
            assert int(result[2]) == int(case["accepted"])
        if not int(result[2]):
            assert float(case["residual"][int(result[0])]) > 0


def test_error_statuses_are_reported_not_raised_on_device():
    vocab = 8
    target = torch.zeros(2, vocab)
    draft = torch.zeros(2, vocab)
    draft[0, 3] = -2000.0
    args = [torch.tensor([0, 2], dtype=torch.int32), torch.tensor([[0, 3]]), torch.tensor([5]),
            torch.tensor([1.0]), torch.tensor([0.5, 0.0]), torch.tensor([0.5])]
    _, status = rlt.accept_rejection(target.cuda(), draft.cuda(), *[a.cuda() for a in args])
    assert status.tolist() == [1]
    with pytest.raises(ValueError, match="zero proposal"):
        rlt.raise_for_status(status.tolist())
    target[0, 0] = float("nan")
    draft[0, 3] = 0.0
    _, status = rlt.accept_rejection(target.cuda(), draft.cuda(), *[a.cuda() for a in args])
    assert status.tolist() == [3]


def test_pipeline_shift_matches_every_reference_step(golden):
    data = golden("pipeline.pt")
    for dtype in (torch.float32, torch.bfloat16):
        for step in data["steps"]:
            before, after = step["before"], step["after"]
            n = before["tokens"].shape[0]
            state = rlt.PipelineState(
                tokens=before["tokens"].cuda(), depths=before["depths"].cuda(), candidates=before["candidates"].cuda(),
                active=before["active"].cuda(), hidden=before["hidden"].to(dtype).cuda(), token=before["token"].cuda(),
                position=before["position"].cuda())
            widths = step["widths"]
            row_starts = torch.zeros(n, dtype=torch.int32)
            row_starts[1:] = widths.cumsum(0)[:-1].int()
            result = rlt.pipeline_shift(state, widths.cuda(), row_starts.cuda(), step["choices"].cuda(),
                                        step["step_hidden"].to(dtype).cuda(), data["limits"].cuda(),
                                        draft_loops=data["draft_loops"], target_loops=data["target_loops"])
            assert torch.equal(result.cpu().flatten(), after["result"])
            for key in ("tokens", "depths", "candidates", "active", "token", "position"):
                assert torch.equal(getattr(state, key).cpu(), after[key]), key
            assert torch.equal(state.hidden.cpu(), after["hidden"].to(dtype))


def _padded_round(n, k, vocab, seed):
    """A round in the fixed shape a graph needs: every request owns k + 1 rows, of which only its
    first counts[i] are real (some requests have none); the rest hold garbage that must never be read."""
    g = torch.Generator().manual_seed(seed)
    width = k + 1
    counts = torch.randint(0, width + 1, (n,), generator=g).int()
    counts[0], counts[1] = 0, width
    cu = (torch.arange(n + 1) * width).int()
    target = torch.randn(n * width, vocab, generator=g) * 3
    draft = target + torch.randn(n * width, vocab, generator=g) * 0.5
    tokens = torch.randint(0, vocab, (n, width), generator=g)
    targets = target.argmax(-1).view(n, width)
    tokens[:, 1:] = torch.where(torch.rand(n, k, generator=g) < 0.6, targets[:, :-1], tokens[:, 1:])
    real = torch.arange(width)[None, :] < counts[:, None]
    target[~real.reshape(-1)] = float("nan")                     # padding rows: poison
    draft[~real.reshape(-1)] = float("nan")
    starts = torch.randint(1, 3000, (n,), generator=g)
    slots = torch.randperm(2 * n, generator=g)[:n]
    return dict(counts=counts, cu=cu, target=target, draft=draft, tokens=tokens, starts=starts, slots=slots, g=g,
                width=width)


def test_fixed_shape_greedy_round_with_padding_rows_matches_the_compact_round():
    n, k, vocab = 23, 4, 2048
    r = _padded_round(n, k, vocab, 5)
    want_slots = torch.full((2 * n, 2), -9, dtype=torch.int64)
    want = oracle.accept_greedy(r["target"], r["cu"], r["tokens"], r["starts"], r["slots"], want_slots, r["counts"])
    got_slots = torch.full((2 * n, 2), -9, dtype=torch.int64).cuda()
    got = rlt.accept_greedy(r["target"].cuda(), r["cu"].cuda(), r["tokens"].cuda(), r["starts"].cuda(), r["slots"].cuda(),
                            got_slots, row_counts=r["counts"].cuda()).cpu()
    assert torch.equal(got, want) and torch.equal(got_slots.cpu(), want_slots)
    # the same requests as a compact round (the reference's layout): same decisions, padding rows are -1
    rows, width = n * r["width"], r["width"]
    keep = (torch.arange(width)[None, :] < r["counts"][:, None]).reshape(-1)
    cu = torch.zeros(n + 1, dtype=torch.int32)
    cu[1:] = r["counts"].cumsum(0)
    live = r["counts"] > 0
    compact = oracle.accept_greedy(r["target"][keep], cu, r["tokens"], r["starts"])
    total = int(cu[-1])
    assert torch.equal(got[:rows][keep], compact[:total]) and bool((got[:rows][~keep] == -1).all())
    assert torch.equal(got[rows:rows + n][live], compact[total:total + n][live])
    assert torch.equal(got[rows + n:][live], compact[total + n:][live])
    # a request without rows is left alone: nothing accepted, position unchanged, slot untouched
    idle = ~live
    assert bool((got[rows:rows + n][idle] == 0).all()) and torch.equal(got[rows + n:][idle], r["starts"][idle])
    assert bool((got_slots.cpu()[r["slots"][idle]] == -9).all())


def test_fixed_shape_rejection_round_with_padding_rows_matches_the_oracle():
    n, k, vocab = 19, 3, 4096
    r = _padded_round(n, k, vocab, 8)
    g, width = r["g"], r["width"]
    temperature = torch.full((n,), 0.8)
    temperature[::5] = 0.0
    u_accept, u_final = torch.rand(n * width, generator=g), torch.rand(n, generator=g)
    top_k = torch.full((n,), -1, dtype=torch.int32)       # filters off (their arrays still travel the padded path)
    top_p = torch.ones(n)
    want_slots = torch.full((2 * n, 2), -9, dtype=torch.int64)
    want, want_status = oracle.accept_rejection(r["target"], r["draft"], r["cu"], r["tokens"], r["starts"], temperature,
                                                u_accept, u_final, r["slots"], want_slots, top_k, top_p, r["counts"])
    got_slots = torch.full((2 * n, 2), -9, dtype=torch.int64).cuda()
    status = torch.full((n,), 7, dtype=torch.int32).cuda()
    workspace = torch.empty(rlt.load_library().rlt_accept_rejection_workspace_bytes(n * width), dtype=torch.uint8).cuda()
    got, got_status = rlt.accept_rejection(
        r["target"].cuda(), r["draft"].cuda(), r["cu"].cuda(), r["tokens"].cuda(), r["starts"].cuda(), temperature.cuda(),
        u_accept.cuda(), u_final.cuda(), r["slots"].cuda(), got_slots, None, top_k.cuda(), top_p.cuda(),
        row_counts=r["counts"].cuda(), status=status, workspace=workspace)
    assert got_status is status
    assert torch.equal(got_status.cpu(), want_status) and int(want_status.abs().sum()) == 0   # NaN padding never read
    assert torch.equal(got.cpu(), want) and torch.equal(got_slots.cpu(), want_slots)


def test_a_failed_request_keeps_its_slot_and_misuse_of_result_is_refused():
    vocab = 8
    target, draft = torch.zeros(2, vocab), torch.zeros(2, vocab)
    draft[0, 3] = -2000.0                                          # zero proposal probability for the draft
    slot_values = torch.tensor([[11, 12], [13, 14]]).cuda()
    args = [torch.tensor([0, 2], dtype=torch.int32), torch.tensor([[0, 3]]), torch.tensor([5]),
            torch.tensor([1.0]), torch.tensor([0.5, 0.0]), torch.tensor([0.5])]
    _, status = rlt.accept_rejection(target.cuda(), draft.cuda(), *[a.cuda() for a in args], torch.tensor([1]).cuda(),
                                     slot_values)
    assert status.tolist() == [1] and slot_values.tolist() == [[11, 12], [13, 14]]
    cuda_args = [a.cuda() for a in args]
    for bad in (torch.zeros(3, dtype=torch.int64).cuda(), torch.zeros(8, dtype=torch.int32).cuda()):
        with pytest.raises(ValueError, match="result"):
            rlt.accept_rejection(target.cuda(), draft.cuda(), *cuda_args, result=bad)
        with pytest.raises(ValueError, match="result"):
            rlt.accept_greedy(target.cuda(), cuda_args[0], cuda_args[1], cuda_args[2], result=bad)


def test_round_uniforms_match_the_oracle_and_are_per_request_streams():
    seeds = torch.tensor([0, 1, 2 ** 62 + 5, 1, 77])
    rounds = torch.tensor([0, 3, 9, 4, 2 ** 40])
    got = rlt.round_uniforms(seeds.cuda(), rounds.cuda(), 7)
    want = oracle.round_uniforms(seeds, rounds, 7)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)
        assert float(b.min()) >= 0.0 and float(b.max()) < 1.0
    # the same (seed, round) gives the same uniforms whatever else is in the batch
    alone = rlt.round_uniforms(seeds[3:4].cuda(), rounds[3:4].cuda(), 7)
    assert torch.equal(alone[0][0], got[0][3]) and torch.equal(alone[1][0], got[1][3]) and alone[2][0] == got[2][3]
    assert not torch.equal(got[0][1], got[0][3])                  # another round of the same request differs
