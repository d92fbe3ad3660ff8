"""The speculative runner on the GPU: the reference's runner contract, device-resident rounds, whole
rounds replayed from CUDA graphs, and a bf16 model with Ouro-shaped heads against the reference's
Torch execution.

Goldens: tests/golden/decode.pt (the reference engine's tokens and counters, fp32) and
tests/golden/bf16_model.pt (hidden states and logits of the reference's serial bf16 execution with
128-wide heads and 16-token pages, tests/golden/make_golden_bf16_model.py).
"""

import pytest
import torch

import vllm_rlt_b200 as rlt

pytestmark = pytest.mark.gpu


def build(case, dtype=torch.float32):
    config = rlt.LoopedLMConfig(**case["config"])
    return rlt.LoopedLM(config, rlt.seeded_state_dict(config, case["seed"]), "cuda", dtype)


def open_session(case, *, cuda_graphs, in_flight, temperature=0.0, max_tokens=None):
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"], cuda_graphs=cuda_graphs)
    session = decoder.open(case["prompts"], max_tokens or case["max_tokens"], num_speculative_tokens=case["k"],
                           draft_loops=case["draft_loops"], target_loops=case["target_loops"], temperature=temperature,
                           in_flight=in_flight)
    return decoder, session


# ---- the runner boundary ------------------------------------------------------------------------
def test_submit_returns_a_ticket_and_collect_a_model_runner_output(golden):
    case = golden("decode.pt")["config1"]
    decoder, session = open_session(case, cuda_graphs=False, in_flight=1)
    runner = decoder.runner
    batch = decoder._schedule(session.requests, case["k"], False)
    assert [s.token_count for s in batch.requests] == [case["k"] + 1] * 4
    assert [s.token_start for s in batch.requests] == [len(p) for p in case["prompts"]]
    ticket = runner.submit(batch)
    decoder._after_submission(batch, False)
    assert ticket.has_result
    output = ticket.collect()
    assert ticket.ready() and ticket.collect() is output
    assert isinstance(output, rlt.ModelRunnerOutput) and len(output.speculative) == 4
    for request, result, frontier, want in zip(session.requests, output.speculative, output.frontiers, case["tokens"]):
        assert isinstance(result, rlt.SpeculativeResult)
        assert len(result.token_ids) == result.accepted_count + 1
        assert result.token_ids == want[1:1 + len(result.token_ids)]          # the reference's next tokens
        assert frontier == len(request.prompt_token_ids) + len(result.token_ids)
    stats = runner.stats
    assert (stats.rounds, stats.drafted_tokens, stats.verified_rows) == (4, 4 * case["k"], 4 * (case["k"] + 1))
    # a finished request gives its slot back; a new generation of the same id may take one again
    free = len(runner.free_slots)
    runner.release(session.requests[0])
    assert len(runner.free_slots) == free + 1 and session.requests[0].request_id not in runner.states
    torch.cuda.synchronize()


def test_misuse_raises_before_anything_is_launched(golden):
    case = golden("decode.pt")["tiny_k3"]
    decoder, session = open_session(case, cuda_graphs=False, in_flight=1)
    runner, request = decoder.runner, session.requests[0]
    with pytest.raises(ValueError):
        runner.submit(rlt.SchedulerOutput("speculative", []))
    with pytest.raises(ValueError):
        runner.submit(rlt.SchedulerOutput("speculative", [rlt.ScheduledRequest(request, request.position, 0)]))
    with pytest.raises(ValueError):                                  # a span beyond the reserved pages
        runner.submit(rlt.SchedulerOutput("speculative", [rlt.ScheduledRequest(request, 10 ** 6, 2)]))
    with pytest.raises(ValueError):                                  # more rows than k + 1
        runner.submit(rlt.SchedulerOutput("speculative", [rlt.ScheduledRequest(request, request.position, case["k"] + 2)]))
    span = rlt.ScheduledRequest(request, request.position, 1)
    tickets = [runner.submit(rlt.SchedulerOutput("speculative", [span])) for _ in range(2)]
    with pytest.raises(RuntimeError, match="buffers exhausted"):     # at most two rounds in flight
        runner.submit(rlt.SchedulerOutput("speculative", [span]))
    for ticket in tickets:
        ticket.collect()
    other = rlt.Request(request.request_id, request.prompt_token_ids, request.sampling_params, [1])
    with pytest.raises(RuntimeError, match="reused before retirement"):
        runner.submit(rlt.SchedulerOutput("speculative", [rlt.ScheduledRequest(other, other.position, 1)]))
    torch.cuda.synchronize()


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_two_rounds_are_submitted_without_reading_the_device(golden, monkeypatch, cuda_graphs):
    # the reference's own check of its device-resident runner (tests/test_async_speculative.py:124-171
    # there): no Tensor.item / tolist while two consecutive rounds are submitted; the second round starts
    # from the token and position the first one left in the device slots
    case = golden("decode.pt")["config1"]
    decoder, session = open_session(case, cuda_graphs=cuda_graphs, in_flight=2)
    if cuda_graphs:
        assert decoder.runner._rounds, "the round graphs are captured when the session opens"

    def forbidden(*args, **kwargs):
        raise AssertionError("the device was read during a submission")

    with monkeypatch.context() as patch:
        patch.setattr(torch.Tensor, "item", forbidden)
        patch.setattr(torch.Tensor, "tolist", forbidden)
        assert session.submit_round() and session.submit_round()
        assert not session.submit_round()                            # two rounds are the limit
    assert len(session.pending) == 2
    assert session.collect_round() and session.collect_round()
    for request, want in zip(session.requests, case["tokens"]):
        got = request.generated_token_ids
        assert len(got) >= 3 and got == want[:len(got)]
    session.run()
    session.close()
    assert [r.generated_token_ids[:case["max_tokens"]] for r in session.requests] == case["tokens"]
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", ["tiny_k3", "tiny_k1_draft1", "config1"])
@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_two_rounds_in_flight_give_the_reference_tokens(golden, name, cuda_graphs):
    case = golden("decode.pt")[name]
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"], cuda_graphs=cuda_graphs)
    tokens = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                              draft_loops=case["draft_loops"], target_loops=case["target_loops"], in_flight=2)
    assert tokens == case["tokens"]
    assert decoder.stats.committed_tokens == case["stats"]["committed"]


def test_a_round_replayed_from_its_graph_equals_the_eager_round_bit_for_bit():
    config = rlt.LoopedLMConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=128, rope_theta=10000.0)
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 5), "cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(1, 512, (n,), generator=g).tolist() for n in (40, 3, 17, 70, 9)]
    results = []
    for graphs, temperature in ((False, 0.0), (True, 0.0), (False, 0.7), (True, 0.7)):
        # 5 requests padded to 8 in both modes, so the GEMMs see the same shapes
        decoder = rlt.SelfSpeculativeDecoder(model, cuda_graphs=graphs, capture_sizes=[8])
        tokens = decoder.generate(prompts, 14, num_speculative_tokens=3, temperature=temperature, seed=5, in_flight=2)
        results.append((tokens, decoder.stats.accepted_tokens, decoder.stats.committed_tokens))
        assert model.attention.last_status()["error"] == 0
    assert results[0] == results[1]       # greedy: eager == graph
    assert results[2] == results[3]       # sampled: the same uniforms, the same tokens
    assert results[0][0] != results[2][0]
    assert all(len(t) == 14 for t in results[2][0])


def test_sampled_and_greedy_requests_share_a_round_and_streams_are_per_request(golden):
    # request i draws from its own counter-based stream: what it generates does not depend on which
    # other requests share its rounds (fp32, so the GEMM rows are batch independent too)
    case = golden("decode.pt")["config1"]
    model = build(case)

    def run(indices, temperatures):
        decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
        kv = decoder._allocate([case["prompts"][i] for i in indices], [32 + 24 + 5] * len(indices))
        first = decoder._prefill(kv, [case["prompts"][i] for i in indices])
        requests = [rlt.Request(str(j), case["prompts"][i], rlt.SamplingParams(max_tokens=24, temperature=t, seed=100 + i), [f])
                    for j, (i, t, f) in enumerate(zip(indices, temperatures, first))]
        runner = rlt.B200SpeculativeRunner(model, kv, rlt.SpeculativeConfig(4), max_num_seqs=len(indices), cuda_graphs=False)
        from vllm_rlt_b200.decoder import DecodeSession
        session = DecodeSession(decoder, runner, requests, 4, 1)
        session.run()
        session.close()
        return [r.generated_token_ids for r in requests]

    together = run([0, 1, 2, 3], [0.0, 0.9, 0.0, 0.9])
    assert together[0] == case["tokens"][0][:24] and together[2] == case["tokens"][2][:24]   # greedy ones: golden
    alone = run([1], [0.9])
    assert alone[0] == together[1]
    assert together[1] != case["tokens"][1][:24]


def test_pipeline_state_can_be_suspended_and_restored(golden):
    case = golden("decode.pt")["config1"]
    model = build(case)
    decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
    config = rlt.SpeculativeConfig(case["k"], 2, 4, mode="pipeline")
    kv = decoder._allocate(case["prompts"], [len(p) + case["max_tokens"] + 4 for p in case["prompts"]])
    requests = decoder._requests(case["prompts"], decoder._prefill(kv, case["prompts"]), case["max_tokens"], 0.0, -1, 1.0, 0)
    runner = rlt.B200SpeculativeRunner(model, kv, config, max_num_seqs=4, cuda_graphs=False)
    from vllm_rlt_b200.decoder import DecodeSession
    session = DecodeSession(decoder, runner, requests, case["k"], 1)
    for _ in range(9):
        assert session.submit_round() and session.collect_round()
    victim = requests[2]
    snapshot = runner.snapshot_pipeline(victim, "cpu")
    assert snapshot is not None and snapshot["hidden"].device.type == "cpu"
    runner.release(victim)
    assert runner.snapshot_pipeline(victim, "cpu") is None
    runner.restore_pipeline(victim, snapshot)
    with pytest.raises(RuntimeError):
        runner.restore_pipeline(victim, snapshot)                    # already live again
    session.run()
    session.close()
    assert [r.generated_token_ids[:case["max_tokens"]] for r in requests] == case["tokens"]


# ---- a bf16 model on the tiled kernels against the reference's Torch execution ---------------------
def test_bf16_model_with_128_wide_heads_matches_the_reference_torch_execution(golden):
    # the bounds of the reference's own bf16 check of speculative rounds against serial replay
    # (tests/test_speculative.py:151,181 there): atol 0.08 / rtol 0.04 per element, logits within 0.025
    case = golden("bf16_model.pt")
    config = rlt.LoopedLMConfig(**case["config"])
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, case["seed"]), "cuda", torch.bfloat16)
    sequences, block, tail = case["sequences"], case["block"], 5
    kv = rlt.PagedKV.allocate(model, [len(s) + 1 for s in sequences], block)
    # 1. the prompt part of every sequence, packed, through every loop (the tcgen05 prompt kernel)
    heads = [len(s) - tail for s in sequences]
    requests = torch.tensor([i for i, n in enumerate(heads) for _ in range(n)], device="cuda")
    positions = torch.tensor([j for n in heads for j in range(n)], device="cuda")
    tokens = torch.tensor([t for s, n in zip(sequences, heads) for t in s[:n]], device="cuda")
    cu = torch.tensor([0] + torch.tensor(heads).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    context = torch.tensor(heads, dtype=torch.int32, device="cuda")
    hidden = model.prelude(tokens)
    prompt_hidden = []
    for depth in range(config.total_ut_steps):
        tables = kv.tables[:, depth]
        blocks = tables[requests].gather(1, (positions // block)[:, None]).squeeze(1).long()
        hidden = model.recurrent(hidden, positions, kv.key, kv.value, blocks, positions % block, tables.contiguous(),
                                 context, packed=(cu, max(heads)))
        prompt_hidden.append(hidden)
    # 2. the last five tokens of every sequence as one verification group per request and depth plane
    #    (the grouped TMA / tensor-core verify kernel; every row attends to the prompt and to its siblings)
    requests = torch.tensor([i for i in range(len(sequences)) for _ in range(tail)], device="cuda")
    positions = torch.tensor([n + j for n in heads for j in range(tail)], device="cuda")
    hidden = model.prelude(torch.tensor([t for s in sequences for t in s[-tail:]], device="cuda"))
    tail_hidden = []
    for depth in range(config.total_ut_steps):
        blocks, offsets, tables, lengths = kv.addressing(requests, positions, depth)
        hidden = model.recurrent(hidden, positions, kv.key, kv.value, blocks, offsets, tables, lengths)
        tail_hidden.append(hidden)
    logits = model.coda(hidden)
    status = model.attention.last_status()
    assert status["error"] == 0 and status["items"] == len(sequences) * config.num_key_value_heads   # one group per request
    worst = 0.0
    for i, (n, want_hidden, want_logits) in enumerate(zip(heads, case["hidden"], case["logits"])):
        first = int(cu[i])
        for depth in range(config.total_ut_steps):
            torch.testing.assert_close(prompt_hidden[depth][first:first + n].float().cpu(), want_hidden[depth][:n].float(),
                                       atol=0.08, rtol=0.04)
            torch.testing.assert_close(tail_hidden[depth][i * tail:(i + 1) * tail].float().cpu(),
                                       want_hidden[depth][n:].float(), atol=0.08, rtol=0.04)
        got, want = logits[i * tail:(i + 1) * tail].float().cpu(), want_logits[n:].float()
        torch.testing.assert_close(got, want, atol=0.08, rtol=0.04)
        worst = max(worst, float((got - want).abs().max()) / float(want.abs().max()))
    assert worst < 2e-2          # logits within 2e-2 relative (of the largest logit) for bf16


def test_an_engine_reuses_its_pool_runner_and_graphs_for_the_next_requests(golden):
    # one reserved pool, one runner, graphs captured once; two different sets of requests decoded one after the
    # other give what a fresh engine gives for each (stale K/V of the first set is never read by the second)
    case = golden("decode.pt")["config1"]
    model = build(case)
    k, block = case["k"], case["block"]
    first, second = case["prompts"][:3], [p[:20] for p in case["prompts"][1:]] + [case["prompts"][0][5:]]
    fresh = []
    for prompts in (first, second):
        fresh.append(rlt.SelfSpeculativeDecoder(model, block=block).generate(prompts, 40, num_speculative_tokens=k))
    pages = -(-(32 + 40 + k + 1) // block)
    kv = rlt.PagedKV.reserve(model, 4 * pages * 4, 4, pages, block)
    runner = rlt.B200SpeculativeRunner(model, kv, rlt.SpeculativeConfig(k), max_num_seqs=4, cuda_graphs=True,
                                       capture_sizes=[2, 4])
    captured = None
    for prompts, want in zip((first, second), fresh):
        decoder = rlt.SelfSpeculativeDecoder(model, block=block, cuda_graphs=True)
        session = decoder.open(prompts, 40, num_speculative_tokens=k, kv=kv, runner=runner, in_flight=2)
        session.run()
        session.close()
        assert [r.generated_token_ids[:40] for r in session.requests] == want
        assert not runner.states
        graphs = {key: id(r.graph) for key, r in runner._rounds.items()}
        assert captured is None or graphs == captured          # nothing was captured again
        captured = graphs
    with pytest.raises(ValueError):                            # more requests than the pool's tables hold
        rlt.SelfSpeculativeDecoder(model, block=block).open(case["prompts"] * 2, 8, num_speculative_tokens=k, kv=kv, runner=runner)
