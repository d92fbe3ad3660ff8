"""The host logic of the speculative runner and of the engine loop around it, on CPU.

The CUDA kernels have no CPU form, so here every kernel entry the runner and the model call is replaced
by the CPU oracle's function of the same name (test infrastructure; the product never does this), CUDA
events and pinned memory by stand-ins, and the looped LM runs its tensor-expression path in fp32.  What is
under test is everything else: fixed-shape rounds with padding rows, slot state carried from round to
round, spans and placeholders, one or two rounds in flight, the wire record, pipeline mode.  The goldens
are the reference engine's tokens and counters (tests/golden/decode.pt).
"""

import contextlib

import pytest
import torch

import vllm_rlt_b200 as rlt
from oracle import oracle
from vllm_rlt_b200 import _capi, decoder as decoder_module, kv_cache, looped_lm, runner as runner_module


class _Event:
    def __init__(self, *args, **kwargs):
        pass

    def record(self, *args):
        pass

    def query(self):
        return True

    def synchronize(self):
        pass


class _HostBuffer:
    def __init__(self, plan_elements, wire_elements):
        self.plan = torch.empty(plan_elements, dtype=torch.int64)
        self.wire = torch.empty(wire_elements, dtype=torch.int64)
        self.leased, self.done = False, None


class _Library:
    @staticmethod
    def rlt_accept_rejection_workspace_bytes(rows):
        return 64


class _Attention:
    @contextlib.contextmanager
    def shared_plan(self):
        yield self

    def __call__(self, q, key, value, tables, lengths):
        return oracle.paged_attention(q.contiguous(), key, value, tables.clamp_min(0), lengths)

    def prefill(self, q, key, value, tables, lengths, cu, longest):
        return oracle.paged_attention(q.contiguous(), key, value, tables.clamp_min(0), lengths, cu)


def _accept_greedy(logits, cu, tokens, starts, slots=None, slot_values=None, result=None, row_counts=None):
    out = oracle.accept_greedy(logits.contiguous(), cu, tokens, starts.contiguous(), slots.contiguous(), slot_values,
                               row_counts)
    result[: out.numel()] = out
    return result


def _accept_rejection(target, draft, cu, tokens, starts, temperature, u_accept, u_final, slots=None, slot_values=None,
                      result=None, top_k=None, top_p=None, row_counts=None, status=None, workspace=None):
    out, codes = oracle.accept_rejection(target.contiguous(), draft.contiguous(), cu, tokens, starts.contiguous(),
                                         temperature.contiguous(), u_accept.contiguous(), u_final.contiguous(),
                                         slots.contiguous(), slot_values, top_k.contiguous(), top_p.contiguous(), row_counts)
    result[: out.numel()] = out
    status.copy_(codes)
    return result, status


def _rollback(starts, emitted, tables, block, refcounts=None, **unused):
    return kv_cache.RollbackResult(*oracle.rollback(starts.contiguous(), emitted.contiguous(), tables.contiguous(), block,
                                                    refcounts=refcounts))


def _pipeline_shift(state, widths, row_starts, choices, step_hidden, limits, *, draft_loops, target_loops, result=None):
    fields = dict(tokens=state.tokens, depths=state.depths, candidates=state.candidates, active=state.active.to(torch.uint8),
                  hidden=state.hidden, token=state.token, position=state.position)
    fields = {name: t.contiguous() for name, t in fields.items()}
    out = oracle.pipeline_shift(fields, widths.contiguous(), row_starts.contiguous(), choices.contiguous(), step_hidden,
                                limits.contiguous(), draft_loops, target_loops)
    for name, t in fields.items():
        setattr(state, name, t.bool() if name == "active" else t)
    return out.view(-1, 6)


@pytest.fixture
def on_cpu(monkeypatch):
    """Everything CUDA-specific replaced for the duration of one test."""
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "stream", lambda stream: contextlib.nullcontext())
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda self: self)
    monkeypatch.setattr(runner_module, "_HostBuffer", _HostBuffer)
    monkeypatch.setattr(_capi, "load", lambda: _Library())
    monkeypatch.setattr(looped_lm, "kv_write", lambda kc, vc, k, v, blocks, offsets, write_mask=None, active_rows=None:
                        oracle.kv_write(kc, vc, k.contiguous(), v.contiguous(), blocks, offsets, write_mask))
    monkeypatch.setattr(looped_lm, "silu_and_mul", lambda gate, up: oracle.silu_and_mul(gate.contiguous(), up.contiguous()))
    argmax = lambda logits: oracle.argmax_rows(logits.contiguous())
    monkeypatch.setattr(runner_module, "argmax_rows", argmax)
    monkeypatch.setattr(decoder_module, "argmax_rows", argmax)
    monkeypatch.setattr(runner_module, "accept_greedy", _accept_greedy)
    monkeypatch.setattr(runner_module, "accept_rejection", _accept_rejection)
    monkeypatch.setattr(runner_module, "sample_rows", lambda logits, t, u, top_k=None, top_p=None: oracle.sample_rows(
        logits.contiguous(), t.contiguous(), u.contiguous(), top_k.contiguous(), top_p.contiguous()))
    monkeypatch.setattr(runner_module, "round_uniforms", oracle.round_uniforms)
    monkeypatch.setattr(runner_module, "rollback", _rollback)
    monkeypatch.setattr(runner_module, "pipeline_shift", _pipeline_shift)


def build(case):
    config = rlt.LoopedLMConfig(**case["config"])
    return rlt.LoopedLM(config, rlt.seeded_state_dict(config, case["seed"]), "cpu", torch.float32, attention=_Attention(),
                        fused=False)


def generate(case, **options):
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"], capture_sizes=options.pop("capture_sizes", None))
    tokens = decoder.generate(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                              draft_loops=case["draft_loops"], target_loops=case["target_loops"], **options)
    return tokens, decoder.stats


@pytest.mark.parametrize("name", ["tiny_k3", "tiny_k1_draft1"])
def test_one_round_in_flight_reproduces_the_reference_tokens_and_counters(golden, on_cpu, name):
    case = golden("decode.pt")[name]
    tokens, stats = generate(case)
    want = case["stats"]
    assert tokens == case["tokens"]
    assert (stats.rounds, stats.drafted_tokens, stats.accepted_tokens, stats.committed_tokens, stats.verified_rows) == \
        (want["rounds"], want["drafted"], want["accepted"], want["committed"], want["verified_rows"])


def test_two_rounds_in_flight_and_padded_buckets_give_the_same_tokens(golden, on_cpu):
    case = golden("decode.pt")["tiny_k3"]
    tokens, stats = generate(case, in_flight=2, capture_sizes=[7])     # 4 requests in rounds shaped for 7
    assert tokens == case["tokens"] and stats.committed_tokens == case["stats"]["committed"]
    # the second round of a request was submitted before its first was collected: fewer rows near the limits
    assert stats.verified_rows <= case["stats"]["verified_rows"]


def test_sampling_collapses_to_greedy_at_vanishing_temperature_and_pipeline_mode_is_lossless(golden, on_cpu):
    case = golden("decode.pt")["tiny_k3"]
    tokens, _ = generate(case, temperature=1e-5, seed=3)
    assert tokens == case["tokens"]
    decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"])
    piped = decoder.generate_pipeline(case["prompts"], case["max_tokens"], num_speculative_tokens=case["k"],
                                      draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    assert piped == case["tokens"]
    assert decoder.stats.committed_tokens == case["stats"]["committed"]


def test_spans_follow_the_scheduler_rule(on_cpu):
    decoder = rlt.SelfSpeculativeDecoder.__new__(rlt.SelfSpeculativeDecoder)
    params = rlt.SamplingParams(max_tokens=6)
    fresh = rlt.Request("a", [1, 2, 3], params, [9])
    busy = rlt.Request("b", [1, 2], params, [9], num_output_placeholders=5, num_speculative_rounds=1)
    full = rlt.Request("c", [1], params, [9], num_speculative_rounds=2)
    done = rlt.Request("d", [1], params, [9, 9, 9, 9, 9, 9], finished=True)
    batch = decoder._schedule([fresh, busy, full, done], 4, False)
    # min(k + 1, remaining) rows from the committed position; nothing for a request whose placeholders fill its
    # budget, that has two rounds out, or that is finished
    assert [(s.request.request_id, s.token_start, s.token_count) for s in batch.requests] == [("a", 3, 5)]
    decoder._after_submission(batch, False)
    assert (fresh.num_output_placeholders, fresh.num_speculative_rounds, fresh.position) == (5, 1, 8)
    assert decoder._schedule([fresh], 4, False) is None          # its budget is reserved until the round is collected


REFERENCE = __import__("pathlib").Path(__file__).resolve().parents[1] / "baseline" / "_ref"


@pytest.mark.skipif(not (REFERENCE / "vllm_rlt").is_dir(), reason="no reference package under baseline/_ref")
@pytest.mark.parametrize("name", ["tiny_k3", "tiny_k1_draft1"])
def test_the_reference_engine_can_drive_the_runner_in_place_of_its_own(golden, on_cpu, name):
    # the unmodified reference engine (scheduler, KV-cache manager, prompt path) with this runner as its
    # round controller: `Executor(speculation=...)`, `engine.speculative_runner`; the manager's pools and block
    # tables are read through KVCacheManagerView.  The GPU form of this test is in
    # test_gpu_reference_integration.py; here the kernels are the oracle's.
    import sys

    sys.modules.setdefault("vllm_rlt._C", None)
    sys.path.insert(0, str(REFERENCE))
    try:
        from vllm_rlt import CacheConfig, SamplingParams, SpeculativeConfig
        from vllm_rlt.engine.stage_engine import StageEngine
        from vllm_rlt.models import OuroConfig, OuroForCausalLM
    except Exception as error:
        pytest.skip(f"the reference package does not import here: {error}")
    case = golden("decode.pt")[name]
    theirs = OuroForCausalLM(OuroConfig(**case["config"], max_position_embeddings=256, bos_token_id=0, eos_token_id=0))
    state = rlt.seeded_state_dict(rlt.LoopedLMConfig(**case["config"]), case["seed"])
    theirs.load_state_dict({n: state[n] for n in theirs.state_dict()}, strict=True)
    loops = dict(draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    engine = StageEngine(theirs, cache_config=CacheConfig(256, case["block"]), attention_backend="torch",
                         speculative_config=SpeculativeConfig(case["k"], **loops))
    view = rlt.KVCacheManagerView(engine.cache_manager, max_pages=-(-256 // case["block"]))
    runner = rlt.B200SpeculativeRunner(build(case), view, rlt.SpeculativeConfig(case["k"], **loops), max_num_seqs=8,
                                       cuda_graphs=False, report_frontiers=False)

    class Controller:
        stats = runner.stats
        release = staticmethod(runner.release)

        @staticmethod
        def submit(batch):
            for span in batch.requests:
                runner.refresh_tables(span.request)
            return runner.submit(batch)

    engine.speculative_runner = engine.executor.speculation = Controller
    params = SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True)
    for i, prompt in enumerate(case["prompts"]):
        engine.add_request(str(i), list(prompt), params)
    finished = {}
    while engine.has_unfinished_requests():
        for output in engine.step():
            if output.finished:
                finished[output.request_id] = list(output.token_ids)
    assert [finished[str(i)] for i in range(len(case["prompts"]))] == case["tokens"]
    stats, want = runner.stats, case["stats"]
    assert (stats.rounds, stats.drafted_tokens, stats.accepted_tokens, stats.committed_tokens, stats.verified_rows) == \
        (want["rounds"], want["drafted"], want["accepted"], want["committed"], want["verified_rows"])
    assert not runner.states


def test_manager_view_and_delivery_protocols(golden, on_cpu):
    # KVCacheManagerView: pools as they are, a request's tables from its allocation, refusal of tables wider than the
    # runner was sized for.  Delivery counting: a collected ticket counts its own delivery only in the synchronous
    # protocol (report_frontiers=False); in the device-resident one the engine does, and the ticket leaves it alone.
    from types import SimpleNamespace

    allocation = SimpleNamespace(block_tables=[[3, 1], [0, 2, 5]])
    manager = SimpleNamespace(key_cache=torch.zeros(8, 1, 4, 1, 8), value_cache=torch.zeros(8, 1, 4, 1, 8), block_size=4,
                              _get_allocation=lambda rid: allocation)
    view = rlt.KVCacheManagerView(manager, max_pages=3)
    assert view.key is manager.key_cache and view.block == 4 and view.refcounts is None
    assert view.device_tables("r").tolist() == [[3, 1, 0], [0, 2, 5]]
    with pytest.raises(ValueError, match="wider than max_pages"):
        rlt.KVCacheManagerView(manager, max_pages=2).device_tables("r")

    case = golden("decode.pt")["tiny_k3"]
    for frontiers in (True, False):
        decoder = rlt.SelfSpeculativeDecoder(build(case), block=case["block"])
        kv = decoder._allocate(case["prompts"], [len(p) + case["max_tokens"] + 8 for p in case["prompts"]])
        requests = decoder._requests(case["prompts"], decoder._prefill(kv, case["prompts"]), case["max_tokens"], 0.0, -1, 1.0, 0)
        runner = rlt.B200SpeculativeRunner(build(case), kv, rlt.SpeculativeConfig(case["k"], case["draft_loops"], case["target_loops"]),
                                           max_num_seqs=4, cuda_graphs=False, report_frontiers=frontiers)
        batch = decoder._schedule(requests, case["k"], False)
        ticket = runner.submit(batch)
        output = ticket.collect()
        assert (output.frontiers is not None) == frontiers and ticket.retired
        assert [s.delivered for s in ticket.states] == [0 if frontiers else 1] * len(ticket.states)
        assert all(runner.request_ready(r) for r in requests)
        with pytest.raises(RuntimeError, match="different speculative request generation"):
            runner.release(SimpleNamespace(request_id=requests[0].request_id))
        for request in requests:
            runner.release(request)
        assert not runner.states
