"""Token identity of greedy self-speculative decoding on the GPU kernels with the reference engine.

The golden tokens and counters in tests/golden/decode.pt come from the reference's Torch
execution on CPU (tests/golden/make_golden_decode.py): the reference's tiny test architecture
and a small CPU-runnable configuration (2 layers, hidden 256, 4 x 64 MHA, FFN 688, vocab 1024, 4 loops, 4 prompts
of 32 tokens, 64 generated, k = 4 drafts from depth 2 verified at depth 4, greedy, block 16).
The model here is rebuilt from the same seeded weights and decoded (a) natively and (b) with
block self-speculation through kv_write / verify attention / SiLU-and-Mul / accept_greedy /
rollback; both must give the reference's tokens, and (b) the reference's counters.
"""

import pytest
import torch

import vllm_rlt_b200 as rlt

pytestmark = pytest.mark.gpu


def build(case, dtype=torch.float32):
    config = rlt.LoopedLMConfig(**case["config"])
    state = rlt.seeded_state_dict(config, case["seed"])
    return rlt.LoopedLM(config, state, "cuda", dtype)


@pytest.mark.parametrize("name", ["tiny_k3", "tiny_k1_draft1", "config1"])
def test_speculative_and_native_tokens_match_the_reference_engine(golden, name):
    case = golden("decode.pt")[name]
    model = build(case)
    native = rlt.SelfSpeculativeDecoder(model, block=case["block"]).generate_native(case["prompts"], case["max_tokens"])
    assert native == case["tokens"]
    decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
    speculative = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                   draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    assert speculative == case["tokens"]
    stats, want = decoder.stats, case["stats"]
    assert (stats.rounds, stats.drafted_tokens, stats.accepted_tokens, stats.committed_tokens,
            stats.verified_rows) == (want["rounds"], want["drafted"], want["accepted"], want["committed"],
                                     want["verified_rows"])
    torch.cuda.synchronize()


def test_bf16_ouro_shaped_heads_use_the_tiled_kernel_and_agree_with_native():
    # 16-token pages and 128-wide heads route attention through the TMA / tensor-core kernel.
    config = rlt.LoopedLMConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=128, rope_theta=10000.0)
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 5), "cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(1, 512, (n,), generator=g).tolist() for n in (40, 3, 17)]
    native = rlt.SelfSpeculativeDecoder(model).generate_native(prompts, 12)
    decoder = rlt.SelfSpeculativeDecoder(model)
    speculative = decoder.generate(prompts, 12, num_speculative_tokens=4)
    assert model.attention.last_status()["error"] == 0
    assert decoder.stats.committed_tokens == 3 * 11
    # bf16 GEMMs are not batch invariant, so rows verified together may round differently from
    # rows decoded one at a time; greedy tokens still have to agree almost everywhere.
    same = sum(a == b for x, y in zip(native, speculative) for a, b in zip(x, y))
    assert same >= 0.8 * 36


def test_rejection_sampled_decoding_collapses_to_greedy_at_vanishing_temperature(golden):
    # At T -> 0 every distribution is a point mass on its argmax, so drafts sampled from q,
    # the u*q < p tests and the residual / bonus draws must reproduce greedy decoding exactly,
    # whatever the uniforms are: the reference's golden tokens again, through sample_rows and
    # accept_rejection instead of argmax and accept_greedy.
    case = golden("decode.pt")["config1"]
    model = build(case)
    for seed in (0, 7):
        decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
        tokens = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                  draft_loops=case["draft_loops"], target_loops=case["target_loops"],
                                  temperature=1e-5, seed=seed)
        assert tokens == case["tokens"]
        assert decoder.stats.committed_tokens == case["stats"]["committed"]


def test_rejection_sampled_decoding_is_reproducible_and_seed_dependent(golden):
    case = golden("decode.pt")["tiny_k3"]
    model = build(case)

    def run(seed):
        decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
        tokens = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=3, temperature=0.8,
                                  seed=seed)
        return tokens, decoder.stats

    first, stats = run(3)
    again, _ = run(3)
    other, _ = run(4)
    assert first == again and first != other
    assert all(len(t) == case["max_tokens"] for t in first)
    assert all(0 <= x < case["config"]["vocab_size"] for t in first for x in t)
    assert stats.committed_tokens == sum(len(t) - 1 for t in first)
    # the first token of every request comes from the prefill argmax, so it matches greedy
    assert [t[0] for t in first] == [t[0] for t in case["tokens"]]


def test_top_k_one_sampling_is_greedy_and_top_p_restricts_the_emitted_tokens(golden):
    # top_k = 1 leaves a point mass on the argmax at any temperature (tests/test_sampler.py:76-84
    # of the reference pins the same for Sampler.sample), so sampled decoding gives the golden
    # greedy tokens; a tiny top_p does the same through the nucleus filter.
    case = golden("decode.pt")["config1"]
    model = build(case)
    for filters in (dict(top_k=1), dict(top_p=1e-6)):
        decoder = rlt.SelfSpeculativeDecoder(model, block=case["block"])
        tokens = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                  draft_loops=case["draft_loops"], target_loops=case["target_loops"],
                                  temperature=1.3, seed=11, **filters)
        assert tokens == case["tokens"]
    # a wider filter still changes what is sampled
    plain = rlt.SelfSpeculativeDecoder(model, block=case["block"]).generate(
        case["prompts"], 24, num_speculative_tokens=case["k"], temperature=1.3, seed=11)
    narrow = rlt.SelfSpeculativeDecoder(model, block=case["block"]).generate(
        case["prompts"], 24, num_speculative_tokens=case["k"], temperature=1.3, seed=11, top_k=5, top_p=0.9)
    assert plain != narrow


@pytest.mark.parametrize("dtype,tolerance", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
def test_fused_layer_kernels_agree_with_the_tensor_expressions(dtype, tolerance):
    # one recurrent loop with rope_kv_write + sandwich_norm against RMSNorm / RoPE / KV write as
    # separate tensor expressions: same K/V pool contents and hidden state to the dtype's tolerance
    # (the fused path also runs q, k and v as one projection, so the GEMM bits differ).
    config = rlt.LoopedLMConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=128, rope_theta=10000.0)
    state = rlt.seeded_state_dict(config, 9)
    fused = rlt.LoopedLM(config, state, "cuda", dtype)
    plain = rlt.LoopedLM(config, state, "cuda", dtype, fused=False)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(1, 512, (n,), generator=g).tolist() for n in (33, 5, 18)]
    outputs = []
    for model in (fused, plain):
        kv = rlt.PagedKV.allocate(model, [len(p) + 4 for p in prompts], 16)
        requests = torch.tensor([i for i, p in enumerate(prompts) for _ in p], device="cuda")
        positions = torch.tensor([j for p in prompts for j in range(len(p))], device="cuda")
        hidden = model.prelude(torch.tensor([t for p in prompts for t in p], device="cuda"))
        before = hidden.clone()
        blocks, offsets, tables, lengths = kv.addressing(requests, positions, 0)
        out = model.recurrent(hidden, positions, kv.key, kv.value, blocks, offsets, tables, lengths)
        assert torch.equal(hidden, before)                      # the caller's tensor is not the residual stream
        outputs.append((out.float(), kv.key.float(), kv.value.float()))
    (a, ka, va), (b, kb, vb) = outputs
    torch.testing.assert_close(a, b, rtol=tolerance, atol=tolerance)
    torch.testing.assert_close(ka, kb, rtol=tolerance, atol=tolerance)
    torch.testing.assert_close(va, vb, rtol=tolerance, atol=tolerance)


@pytest.mark.parametrize("name", ["tiny_k3", "config1"])
def test_graph_captured_loops_give_the_reference_tokens_and_counters(golden, name):
    # every recurrent loop replayed from a CUDA graph per row bucket (padding rows write no K/V
    # and attend to nothing): the reference engine's tokens and counters again
    case = golden("decode.pt")[name]
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"], cuda_graphs=True)
    speculative = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                   draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    assert speculative == case["tokens"]
    stats, want = decoder.stats, case["stats"]
    assert (stats.rounds, stats.drafted_tokens, stats.accepted_tokens, stats.committed_tokens,
            stats.verified_rows) == (want["rounds"], want["drafted"], want["accepted"], want["committed"],
                                     want["verified_rows"])


def test_graph_replay_equals_the_eager_loop_bit_for_bit():
    config = rlt.LoopedLMConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                num_attention_heads=2, num_key_value_heads=2, head_dim=128, rope_theta=10000.0)
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 5), "cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    lengths = [40, 3, 17, 70, 9]
    results = []
    for graphed in (False, True):
        kv = rlt.PagedKV.allocate(model, [n + 8 for n in lengths], 16)
        loops = rlt.GraphedLoops(model, kv, granularity=32) if graphed else None
        g.manual_seed(4)
        outs = []
        for step in range(3):                                   # growing contexts, three row counts, one bucket reused
            rows = [(i, p) for i, n in enumerate(lengths) for p in range(n if step == 0 else 1)]
            if step:
                rows = [(i, lengths[i] + step - 1) for i in range(len(lengths) - step + 1)]
            requests = torch.tensor([r for r, _ in rows], device="cuda")
            positions = torch.tensor([p for _, p in rows], device="cuda")
            hidden = model.prelude(torch.randint(1, 512, (len(rows),), generator=g).cuda())
            blocks, offsets, tables, lens = kv.addressing(requests, positions, 0)
            if graphed:
                outs.append(loops(hidden, positions, blocks, offsets, tables, lens))
            else:
                outs.append(model.recurrent(hidden, positions, kv.key, kv.value, blocks, offsets, tables, lens))
        results.append((outs, kv.key.clone(), kv.value.clone()))
    (eager, ke, ve), (replayed, kg, vg) = results
    for a, b in zip(eager, replayed):
        assert torch.equal(a, b)
    assert torch.equal(ke, kg) and torch.equal(ve, vg)
    assert model.attention.last_status  # the wrapper stays usable after captures


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["tiny_k3", "config1"])
def test_pipeline_mode_decoding_gives_the_reference_tokens(golden, name, graphs):
    # Pipeline self-speculation (every slot advances d loops per step at its own depth plane, the
    # device state is updated by pipeline_shift) is lossless: the reference engine's greedy tokens —
    # launched from the host, and with every step replayed from the CUDA graph of its batch-size bucket
    # (requests that finish early leave padding rows behind: buckets of 4 and 3 cover 4, 3, 2 and 1 live requests).
    case = golden("decode.pt")[name]
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"], cuda_graphs=graphs,
                                         capture_sizes=[3, 4] if graphs else None)
    tokens = decoder.generate_pipeline(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                       draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    assert tokens == case["tokens"]
    if graphs:
        rounds = decoder.runner._rounds if getattr(decoder, "runner", None) is not None else {}
        assert all(r.graph is not None for key, r in rounds.items() if key[0] == "pipeline")
    stats = decoder.stats
    assert stats.committed_tokens == sum(len(t) - 1 for t in tokens)
    assert 0 <= stats.accepted_tokens <= stats.committed_tokens and stats.drafted_tokens >= stats.accepted_tokens


def test_prefix_reuse_matches_cold_generation(golden):
    # the reference's own check (tests/test_prefix_growth.py:27-45 there): a request that maps an
    # earlier request's complete prompt pages generates what it generates when it computes them
    case = golden("decode.pt")["config1"]
    model = build(case)
    g = torch.Generator().manual_seed(9)
    vocab = case["config"]["vocab_size"]
    base = torch.randint(1, vocab, (50,), generator=g).tolist()
    other = torch.randint(1, vocab, (20,), generator=g).tolist()
    prompts = [base, base[:35] + other[:5], list(base), base[:20] + other[5:15], other]
    cold = rlt.SelfSpeculativeDecoder(model, block=16)
    want = cold.generate(prompts, 24, num_speculative_tokens=4)
    assert cold.stats.prefix_hit_tokens == 0
    warm = rlt.SelfSpeculativeDecoder(model, block=16, prefix_caching=True)
    got = warm.generate(prompts, 24, num_speculative_tokens=4)
    assert got == want
    assert warm.stats.prefix_hit_tokens == 32 + 48 + 16
    assert warm.stats.prompt_tokens_computed == sum(len(p) for p in prompts) - 96
    assert rlt.SelfSpeculativeDecoder(model, block=16, prefix_caching=True).generate_native(prompts, 24) == want
    torch.cuda.synchronize()
