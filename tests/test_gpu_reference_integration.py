"""The B200 kernels plugged into the vllm-rlt reference itself.

Runs only where an UNMODIFIED copy of the reference package is importable from `baseline/_ref/`
(`python -m pip install --no-deps --no-build-isolation --target baseline/_ref <reference checkout>`; the
directory is not part of this repository).  The test then does what a maintainer of the reference would do
to adopt the kernels: one more backend name in `validate_backend_name` / `_create_explicit`
that wraps `B200PagedAttention` in the reference's OWN `AttentionBackend` / `BackendCapabilities` classes, and
`register_torch_op("vllm_rlt")` so that `torch.ops.vllm_rlt.silu_and_mul` dispatches CUDA tensors to the B200
kernel — and runs the reference's engine (its scheduler, KV-cache manager, speculative runner and model code,
on the GPU) to the golden tokens of its CPU run (tests/golden/decode.pt).  A second step replaces the
reference's speculative runner by `B200SpeculativeRunner` under the same unmodified engine.
"""

import dataclasses
import sys
from pathlib import Path

import pytest
import torch

import vllm_rlt_b200 as rlt

REFERENCE = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REFERENCE / "vllm_rlt").is_dir(), reason="no reference package under baseline/_ref")]


@pytest.fixture(scope="module")
def reference():
    """The reference package with its own native extension kept out, so that the only CUDA implementation
    of `torch.ops.vllm_rlt.silu_and_mul` is the one this library registers."""
    sys.modules.setdefault("vllm_rlt._C", None)          # `import vllm_rlt._C` now fails: the op is defined in Python
    sys.path.insert(0, str(REFERENCE))
    try:
        import vllm_rlt
        import vllm_rlt.kernels.activation  # defines the schema + the composite fallback
    except Exception as error:  # missing optional dependency of the reference on this box
        pytest.skip(f"the reference package does not import here: {error}")
    rlt.register_torch_op("vllm_rlt")
    return vllm_rlt


@pytest.fixture
def b200_backend(reference, monkeypatch):
    """The two-line patch of the reference: a backend name and its constructor."""
    from vllm_rlt.attention import backend as backend_module
    from vllm_rlt.core import kv_cache_manager as cache_module

    original = backend_module.validate_backend_name

    def validate(name):
        if name != "b200":
            original(name)

    def explicit(name, device, dtype, head_dim, block_size):
        if name != "b200":
            return create(name, device, dtype, head_dim, block_size)
        ours = rlt.create_backend(device, dtype, head_dim, block_size)
        capabilities = backend_module.BackendCapabilities(**dataclasses.asdict(ours.capabilities))
        return backend_module.AttentionBackend(ours.kernel, capabilities, {"backend": "b200"})

    create = backend_module._create_explicit
    monkeypatch.setattr(backend_module, "validate_backend_name", validate)
    monkeypatch.setattr(cache_module, "validate_backend_name", validate)
    monkeypatch.setattr(backend_module, "_create_explicit", explicit)
    return backend_module


def reference_model(case, dtype=torch.float32):
    from vllm_rlt.models import OuroConfig, OuroForCausalLM

    # The reference allocates its KV pools with torch.empty (core/kv_cache_manager.py:143-145): whatever the caching
    # allocator hands back is what lies behind every context's last token.  Leave it blocks of NaN to hand back.
    for elements in (1 << 18, 1 << 20, 1 << 22, 1 << 24):
        torch.full((elements,), float("nan"), dtype=torch.float32, device="cuda")

    config = OuroConfig(**case["config"], max_position_embeddings=256, bos_token_id=0, eos_token_id=0)
    model = OuroForCausalLM(config)
    state = rlt.seeded_state_dict(rlt.LoopedLMConfig(**case["config"]), case["seed"])
    model.load_state_dict({name: state[name] for name in model.state_dict()}, strict=True)
    return model.to(device="cuda", dtype=dtype)


def run_engine(engine, prompts, params):
    for i, prompt in enumerate(prompts):
        engine.add_request(str(i), list(prompt), params)
    finished = {}
    while engine.has_unfinished_requests():
        for output in engine.step():
            if output.finished:
                finished[output.request_id] = list(output.token_ids)
    return [finished[str(i)] for i in range(len(prompts))]


class RoundControllerOnTheReferenceCache:
    """What the reference's `Executor(speculation=...)` and `StageEngine.speculative_runner` get instead of
    the reference's own `SpeculativeRunner`: `submit(batch) -> ticket`, `release(request)`, `stats`.  The
    reference's KV-cache manager goes on owning the pools and the block tables; the B200 runner reads both
    through `KVCacheManagerView` and is told to look at a request's tables again before each of its rounds."""

    def __init__(self, engine, case, dtype, k, **config):
        self.model = rlt.LoopedLM(rlt.LoopedLMConfig(**case["config"]), engine.model.state_dict(), "cuda", dtype)
        manager = engine.cache_manager
        view = rlt.KVCacheManagerView(manager, max_pages=-(-256 // manager.block_size))
        self.runner = rlt.B200SpeculativeRunner(
            self.model, view, rlt.SpeculativeConfig(k, **config), max_num_seqs=engine.scheduler.config.max_num_seqs,
            cuda_graphs=False, report_frontiers=False)
        self.stats = self.runner.stats
        self.submitted = 0

    def submit(self, batch):
        for span in batch.requests:
            self.runner.refresh_tables(span.request)
        self.submitted += 1
        return self.runner.submit(batch)

    def release(self, request):
        self.runner.release(request)

    def install(self, engine):
        engine.speculative_runner = engine.executor.speculation = self
        return engine


def test_torch_op_of_the_reference_dispatches_to_the_b200_kernel(reference):
    from vllm_rlt.kernels.activation import silu_and_mul

    g = torch.Generator().manual_seed(1)
    gate, up = (torch.randn(37, 5632, generator=g) * 3).bfloat16().cuda(), torch.randn(37, 5632, generator=g).bfloat16().cuda()
    assert torch.equal(silu_and_mul(gate, up), rlt.silu_and_mul(gate, up))
    assert torch.equal(silu_and_mul(gate, up), torch.nn.functional.silu(gate) * up)
    with pytest.raises(RuntimeError, match="contiguous"):          # the B200 entry is what ran: its own check fires
        silu_and_mul(gate[:, ::2], up[:, ::2])


@pytest.mark.parametrize("name", ["config1", "tiny_k3"])
def test_reference_engine_decodes_the_golden_tokens_on_the_b200_backend(reference, b200_backend, golden, name):
    from vllm_rlt import CacheConfig, SamplingParams, SpeculativeConfig
    from vllm_rlt.engine.stage_engine import StageEngine

    case = golden("decode.pt")[name]
    model = reference_model(case)
    params = SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True)
    native = StageEngine(model, cache_config=CacheConfig(256, case["block"]), attention_backend="b200")
    cache = native.cache_manager
    assert type(cache.attention).__module__.startswith("vllm_rlt.attention")       # the reference's adapter class ...
    assert isinstance(cache.attention.kernel, rlt.B200PagedAttention)             # ... around the B200 kernel
    assert cache.attention_info["selected_backend"] == "b200"
    assert run_engine(native, case["prompts"], params) == case["tokens"]
    speculative = StageEngine(model, cache_config=CacheConfig(256, case["block"]), attention_backend="b200",
                              speculative_config=SpeculativeConfig(case["k"], draft_loops=case["draft_loops"],
                                                                   target_loops=case["target_loops"]))
    assert run_engine(speculative, case["prompts"], params) == case["tokens"]
    stats, want = speculative.speculative_runner.stats, case["stats"]
    assert (stats.rounds, stats.drafted_tokens, stats.verified_rows) == (want["rounds"], want["drafted"], want["verified_rows"])
    torch.cuda.synchronize()


@pytest.mark.parametrize("incremental", [False, True])
@pytest.mark.parametrize("name", ["config1", "tiny_k3"])
def test_reference_engine_drives_the_b200_round_controller_to_the_golden_tokens(reference, b200_backend, golden, name, incremental):
    # the reference's scheduler, KV-cache manager, prompt path and token bookkeeping, unmodified, with the
    # B200 runner in the place of its SpeculativeRunner: same tokens, same round statistics
    from vllm_rlt import CacheConfig, SamplingParams, SpeculativeConfig
    from vllm_rlt.engine.stage_engine import StageEngine

    case = golden("decode.pt")[name]
    model = reference_model(case)
    params = SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True)
    loops = dict(draft_loops=case["draft_loops"], target_loops=case["target_loops"])
    # incremental: the manager grows a request's block tables as it decodes (CacheConfig.incremental_allocation), so the
    # runner's copy of them has to follow (`refresh_tables` before every round)
    engine = StageEngine(model, cache_config=CacheConfig(256, case["block"], incremental_allocation=incremental),
                         attention_backend="b200", speculative_config=SpeculativeConfig(case["k"], **loops))
    controller = RoundControllerOnTheReferenceCache(engine, case, torch.float32, case["k"], **loops)
    controller.install(engine)
    assert run_engine(engine, case["prompts"], params) == case["tokens"]
    assert controller.submitted > 0 and not controller.runner.states            # every request was released
    stats, want = controller.stats, case["stats"]
    assert (stats.rounds, stats.drafted_tokens, stats.verified_rows) == (want["rounds"], want["drafted"], want["verified_rows"])
    assert (stats.committed_tokens, stats.accepted_tokens) == (want["committed"], want["accepted"])
    torch.cuda.synchronize()


def test_reference_engine_on_the_tiled_kernel_agrees_with_its_torch_backend(reference, b200_backend):
    # bf16, 128-wide heads, 16-token pages: the reference's model and runner on the TMA / tensor-core kernel
    # against the same engine on its own Torch attention; greedy tokens agree (bf16 rounding may flip a near-tie)
    from vllm_rlt import CacheConfig, SamplingParams, SpeculativeConfig
    from vllm_rlt.engine.stage_engine import StageEngine

    case = dict(config=dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                            num_attention_heads=2, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
                            rope_theta=10000.0, total_ut_steps=4, initializer_range=0.02), seed=21)
    model = reference_model(case, torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(1, 512, (n,), generator=g).tolist() for n in (40, 3, 17)]
    params = SamplingParams(max_tokens=12, ignore_eos=True)
    outputs = {}
    for backend in ("torch", "b200"):
        engine = StageEngine(model, cache_config=CacheConfig(64, 16), attention_backend=backend,
                             speculative_config=SpeculativeConfig(3))
        outputs[backend] = run_engine(engine, prompts, params)
    engine = StageEngine(model, cache_config=CacheConfig(64, 16), attention_backend="b200",
                         speculative_config=SpeculativeConfig(3))
    RoundControllerOnTheReferenceCache(engine, case, torch.bfloat16, 3).install(engine)
    outputs["b200 runner"] = run_engine(engine, prompts, params)
    for name in ("b200", "b200 runner"):
        same = sum(a == b for x, y in zip(outputs["torch"], outputs[name]) for a, b in zip(x, y))
        assert same >= 0.8 * 36, outputs


def test_reference_cache_manager_attends_through_the_b200_window_entry(reference, b200_backend):
    # KVCacheManager.attend(..., window=) reaches `attention.windowed` only on a backend that advertises
    # `sliding_window` (core/kv_cache_manager.py:773-803): the manager on the B200 backend against the same manager
    # on its own Torch kernel, after identical writes (the scene of tests/test_dory.py:409-437, on the GPU)
    from vllm_rlt.core.kv_cache_manager import KVCacheManager

    def manager(backend):
        return KVCacheManager(num_layers=2, num_kv_heads=2, head_dim=8, num_blocks=64, block_size=2, max_loops=2,
                              device="cuda", dtype=torch.float32, backend=backend)

    ours, theirs = manager("b200"), manager("torch")
    assert ours.attention_capabilities.sliding_window and isinstance(ours.attention.kernel, rlt.B200PagedAttention)
    g = torch.Generator().manual_seed(7)
    for cache in (ours, theirs):
        assert cache.allocate("request", 12)
    for position in range(12):
        k, v = torch.randn(1, 2, 8, generator=g).cuda(), torch.randn(1, 2, 8, generator=g).cuda()
        for cache in (ours, theirs):
            cache.write(1, ["request"], [0], [position], k, v)
    query = torch.randn(1, 4, 8, generator=g).cuda()
    for window in (1, 3, 12, 50):
        got = ours.attend(1, ["request"], [0], [11], query, window=window)
        want = theirs.attend(1, ["request"], [0], [11], query, window=window)
        torch.testing.assert_close(got, want, atol=3e-6, rtol=1e-5)
    assert not torch.allclose(ours.attend(1, ["request"], [0], [11], query, window=3),
                              ours.attend(1, ["request"], [0], [11], query))


@pytest.mark.parametrize("mode", ["block", "pipeline"])
@pytest.mark.parametrize("graphs", [False, True])
def test_reference_async_engine_drives_the_b200_runner_with_two_rounds_in_flight(reference, b200_backend, golden, graphs, mode):
    # `ExecutionConfig(async_scheduling=True)`: the reference's engine submits a round ahead of the one it collects,
    # books placeholders at submission, checks every collected round against the device's frontier and counts
    # deliveries itself (engine/stage_engine.py:732-793, core/scheduler.py:1362-1375).  Its AsyncSpeculativeRunner is
    # replaced by B200SpeculativeRunner in its default, device-resident protocol; nothing else changes.
    from vllm_rlt import CacheConfig, ExecutionConfig, SamplingParams, SpeculativeConfig
    from vllm_rlt.engine.stage_engine import StageEngine

    case = golden("decode.pt")["config1"]
    model = reference_model(case)
    loops = dict(draft_loops=case["draft_loops"], target_loops=case["target_loops"], mode=mode)
    engine = StageEngine(model, cache_config=CacheConfig(256, case["block"]), attention_backend="b200",
                         execution_config=ExecutionConfig(async_scheduling=True),
                         speculative_config=SpeculativeConfig(case["k"], **loops))
    assert engine.async_speculative and engine.pipeline_speculative == (mode == "pipeline")
    ours = rlt.LoopedLM(rlt.LoopedLMConfig(**case["config"]), model.state_dict(), "cuda", torch.float32)
    view = rlt.KVCacheManagerView(engine.cache_manager, max_pages=-(-256 // case["block"]))
    runner = rlt.B200SpeculativeRunner(ours, view, rlt.SpeculativeConfig(case["k"], **loops),
                                       max_num_seqs=engine.scheduler.config.max_num_seqs, cuda_graphs=graphs,
                                       compute_stream=engine.model_runner.core_stream)
    engine.speculative_runner = engine.executor.speculation = runner
    in_flight = []
    submit = runner.submit

    def counted(batch):
        ticket = submit(batch)
        in_flight.append(len(engine._pending_speculative) + 1)
        return ticket

    runner.submit = counted
    params = SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True)
    assert run_engine(engine, case["prompts"], params) == case["tokens"]
    assert max(in_flight) == 2 and not runner.states and not engine._pending_speculative
    assert runner.stats.committed_tokens == sum(len(t) - 1 for t in case["tokens"])
    assert all(not buffer.leased for buffer in runner.buffers)
    torch.cuda.synchronize()
