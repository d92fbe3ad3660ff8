"""Benchmark of the self-speculative verify step on B200 (and its CPU baseline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

The contract line measures two things in one process per GPU.

1. Self-speculative decoding of an Ouro-1.4B-shaped model (24 layers, hidden 2048, 16 x 128 MHA,
   SwiGLU 5632, vocab 49152, 4 recurrent loops, random-init bf16): 128 concurrent requests with
   prompts of uniform-random tokens, lengths U[128, 1024], k = 4 drafts from loop depth 2 verified at
   depth 4, rejection sampling at temperature 0.8, through `SelfSpeculativeDecoder` /
   `B200SpeculativeRunner`.  A *step* is one speculative round of the whole batch (5 draft passes of
   128 rows through 2 loops, 2 verify passes of 640 rows, LM head, acceptance, rollback — one CUDA
   graph).  After the prompts are in the cache and the graph exists, W warm-up rounds run, then K
   rounds are timed with CUDA events (`value` = accepted tokens per second; committed tokens per
   second and the acceptance rate beside it), then K more rounds are timed on the host clock from
   `runner.submit(batch)` (Python request objects in) to `ticket.collect()` (Python token lists out):
   `e2e`.  The GEMMs of the model are cuBLAS call sites; every other kernel is this library's.
2. The verify attention alone at the kernel-microbench shape (64 requests, contexts U[512, 4096],
   16 rows per request = 4 tokens x 4 loop depths on a shared plane, 24-layer pool): its CUDA-event
   time per layer call against its algorithmic bytes is the `roofline` block, and its output for a
   few requests is compared with the CPU oracle (`parity`).

With N GPUs every rank is an independent engine replica that decodes the same 128 seeded requests
(no collective on the path); the timed regions are bracketed by a barrier, the step time is the
maximum over ranks and the tokens are summed, so the aggregate depends on step times only.

Other entry points (each prints its own JSON line; none is the contract line above):
    --workload decode [--requests R --output-tokens T --temperature X --k K --eager --prompt-min A --prompt-max B
                       --shared-prefix P --prefix-caching --in-flight F]
                      one complete generation (prompt pass included in `total_seconds`)
    --workload decode --engine reference [--sync]
                      the same requests, weights and output budget through the UNMODIFIED reference engine on the
                      GPU, when a copy of it is importable from baseline/_ref: its own scheduler, runner, Triton
                      attention and CUDA graphs (`ExecutionConfig(async_scheduling=True, cuda_graphs=True)`; greedy
                      only — `--sync` selects its synchronous runner, which also samples) — the same-box comparison;
                      `--adopt attention|runner` plugs this library's attention backend (and speculative runner) into
                      that engine (a backend name and a runner assignment on the reference's side)
    --workload sharded [--total-requests R ...]
                      R requests in total (default 1024, prompts U[256, 2048], 512 output tokens, k = 6, T = 0.8),
                      length-balanced over the ranks and decoded to completion in waves that fit the KV
                      pool: whole-job strong scaling
    --only attention  [--requests --layers --tokens --depths --kv-heads --context-min --context-max --shared-plan]
    --only prefill    [--requests --tokens --kv-heads --eager]   packed causal prefill, TFLOP/s
    --only accept | --only silu                                  the small kernels at the step's shapes
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LAYERS, HEADS, HEAD_DIM, BLOCK, FFN, VOCAB = 24, 16, 128, 16, 5632, 49152
REQUESTS, TOKENS, DEPTHS = 64, 4, 4
TEMPERATURE = 0.8
DECODE_REQUESTS, DECODE_PROMPTS, DECODE_K, DECODE_OUTPUT = 128, (128, 1024), 4, 256
DRAFT_LOOPS, TARGET_LOOPS = 2, 4
METRIC = "accepted tokens/s/GPU, Ouro-1.4B self-spec decode; verify-attn % HBM peak"
# DRAM bytes (read + write) per algorithmic byte of verify_attention_kernel, from an ncu capture of a
# 32-request launch of the same kernel (654.4 + 7.9 MB moved for 653.9 MB algorithmic); traffic grows
# in proportion to the K/V read, so the ratio carries over to a full launch.
ATTENTION_TRAFFIC_RATIO = 1.0128


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class Workload:
    """Seeded synthetic inputs of one replica (one GPU or the CPU sample)."""

    def __init__(self, seed: int, requests: int = REQUESTS, layers: int = LAYERS, device="cpu",
                 tokens: int = TOKENS, depths: int = DEPTHS, kv_heads: int = HEADS, context_range=(512, 4096)):
        g = torch.Generator().manual_seed(seed)
        self.requests, self.layers = requests, layers
        TOKENS, DEPTHS = tokens, depths
        self.kv_heads = kv_heads
        self.contexts = torch.randint(context_range[0], context_range[1] + 1, (requests,), generator=g)
        pages = (self.contexts + BLOCK - 1) // BLOCK
        self.total_pages = int(pages.sum())
        order = torch.randperm(self.total_pages, generator=g).int()
        width = int(pages.max())
        tables = torch.zeros(requests, width, dtype=torch.int32)
        offset = 0
        for i, n in enumerate(pages.tolist()):
            tables[i, :n] = order[offset:offset + n]
            offset += n
        self.request_tables = tables
        rows_per_request = TOKENS * DEPTHS
        # row (depth, t) of a request sees ctx - 3 + t keys; all 16 rows share one table row
        visible = torch.stack([self.contexts - (TOKENS - 1) + t for t in range(TOKENS)], 1)  # [req, tok]
        self.lengths = visible.repeat(1, DEPTHS).reshape(-1).int()
        self.tables = tables.repeat_interleave(rows_per_request, 0).contiguous()
        self.rows = requests * rows_per_request
        positions = (visible - 1).reshape(-1)  # new tokens: one K/V row per (request, token)
        req_of = torch.arange(requests).repeat_interleave(TOKENS)
        self.write_blocks = tables[req_of, (positions // BLOCK)].long()
        self.write_offsets = (positions % BLOCK).long()
        self.kv_rows = requests * TOKENS
        self.seed = seed
        self.device = torch.device(device)
        self.generator = g
        # acceptance inputs: 4 rows per request (3 drafts + bonus row)
        self.accept_rows = requests * TOKENS
        self.cu_rows = (torch.arange(requests + 1) * TOKENS).int()
        self.starts = (self.contexts - TOKENS).long()
        self.slots = torch.randperm(2 * requests, generator=g)[:requests]
        self.temperature = torch.full((requests,), TEMPERATURE)

    def algorithmic_attention_bytes(self) -> int:
        """Each group's K/V once + Q + O + block tables, per layer call."""
        kv = int(self.contexts.sum()) * self.kv_heads * HEAD_DIM * 2 * 2
        qo = self.rows * HEADS * HEAD_DIM * 2 * 2
        tables = int(((self.contexts + BLOCK - 1) // BLOCK).sum()) * 4
        return kv + qo + tables

    def host_inputs(self, pin: bool):
        """Per-step inputs as host tensors (bf16 activations, fp32 logits)."""
        g = self.generator
        def mk(*shape, scale=1.0, dtype=torch.bfloat16):
            t = (torch.randn(*shape, generator=g) * scale).to(dtype)
            return t.pin_memory() if pin else t
        inputs = dict(
            q=mk(self.layers, self.rows, HEADS, HEAD_DIM, scale=0.5),
            k=mk(self.layers, self.kv_rows, HEADS, HEAD_DIM, scale=0.5),
            v=mk(self.layers, self.kv_rows, HEADS, HEAD_DIM, scale=0.5),
            gate=mk(self.layers, self.rows, FFN, scale=3.0),
            up=mk(self.layers, self.rows, FFN),
            target=mk(self.accept_rows, VOCAB, scale=3.0, dtype=torch.float32),
        )
        noise = mk(self.accept_rows, VOCAB, scale=0.5, dtype=torch.float32)
        draft = inputs["target"] + noise
        inputs["draft"] = draft.pin_memory() if pin else draft
        small = dict(tables=self.tables, lengths=self.lengths, write_blocks=self.write_blocks,
                     write_offsets=self.write_offsets, cu_rows=self.cu_rows, starts=self.starts,
                     slots=self.slots, temperature=self.temperature,
                     u_draft=torch.rand(self.accept_rows, generator=g),
                     u_accept=torch.rand(self.accept_rows, generator=g),
                     u_final=torch.rand(self.requests, generator=g),
                     request_tables=self.request_tables[:, None, :].repeat(1, DEPTHS, 1).contiguous())
        for name, t in small.items():
            inputs[name] = t.pin_memory() if pin else t
        return inputs


def combine_ranks(stats, world: int, steps: int, gather=None):
    """Whole-job numbers from per-rank [timed ms, e2e ms, accepted/step, committed/step].

    Replicas are independent, so the job's step time is the slowest rank's (max over ranks) and its
    tokens are the sum over ranks.  `gather(tensor) -> [world, 4]` collects the rows
    (torch.distributed all_gather in a multi-rank run)."""
    if stats.dim() == 2:
        table = stats                                      # already one row per rank
    else:
        table = stats[None] if gather is None or world == 1 else gather(stats)
    max_ms, max_e2e_ms = float(table[:, 0].max()), float(table[:, 1].max())
    accepted, committed = float(table[:, 2].sum()), float(table[:, 3].sum())
    ms_per_step = max_ms / steps
    return {
        "ms_per_step": ms_per_step,
        "e2e_ms_per_step": max_e2e_ms / steps,
        "accepted_per_step": accepted,
        "committed_per_step": committed,
        "accepted_tokens_per_s": accepted / (ms_per_step / 1e3),
        "committed_tokens_per_s": committed / (ms_per_step / 1e3),
        "e2e_accepted_tokens_per_s": accepted / (max_e2e_ms / steps / 1e3),
    }


def all_gather_rows(stats):
    """[4] per rank -> [world, 4] on every rank (any torch.distributed backend)."""
    import torch.distributed as dist

    rows = [torch.zeros_like(stats) for _ in range(dist.get_world_size())]
    dist.all_gather(rows, stats)
    return torch.stack(rows).cpu()


def replica_seed(rank: int) -> int:
    """Every replica draws its own requests: same distribution, different seed."""
    return 1234 + rank


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        try:  # address the GPU by UUID: nvidia-smi indices ignore CUDA_VISIBLE_DEVICES
            index = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
        except Exception:
            pass
        self.index, self.samples, self.process = index, [], None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is None:
            return
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except Exception:
            self.process.kill()
            out = ""
        for line in out.splitlines():
            fields = [x.strip() for x in line.split(",")]
            if len(fields) >= 9:
                self.samples.append(fields)

    def summary(self):
        sm = [float(s[1]) for s in self.samples if len(s) > 2 and s[1].replace(".", "").isdigit()]
        mx = [float(s[2]) for s in self.samples if len(s) > 2 and s[2].replace(".", "").isdigit()]
        reasons = set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            for name, flag in zip(names, s[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def decode_prompts(requests: int, prompt_range, vocab: int, seed: int = 11):
    """Uniform-random token prompts with lengths U[prompt_range] (the same list for a given seed)."""
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(prompt_range[0], prompt_range[1] + 1, (requests,), generator=g).tolist()
    return [torch.randint(1, vocab, (n,), generator=g).tolist() for n in lengths]


def decode_round_bytes(config, stats_before, stats_after, rounds: int, k: int):
    """Algorithmic HBM bytes of `rounds` speculative rounds: every recurrent pass streams the layer
    weights once and, per layer, the K/V of every context it attends to once per request; every LM-head
    call streams lm_head once (k draft calls and one verify call per round).  Activations and logits are
    left out (a few percent)."""
    c = config
    layer_params = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                    + c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    passes = stats_after.loop_passes - stats_before.loop_passes
    context_tokens = stats_after.context_tokens_read - stats_before.context_tokens_read
    weight_bytes = 2.0 * c.num_hidden_layers * layer_params * passes
    kv_bytes = 2.0 * 2 * c.num_key_value_heads * c.head_dim * c.num_hidden_layers * context_tokens
    head_bytes = 2.0 * c.vocab_size * c.hidden_size * (k + 1) * rounds
    return {"weight_bytes": weight_bytes, "kv_bytes": kv_bytes, "lm_head_bytes": head_bytes,
            "total": weight_bytes + kv_bytes + head_bytes}


def launches_per_round(config, k: int, draft_loops: int, target_loops: int, sampled: bool) -> int:
    """Kernels of this library in one round's graph (the cuBLAS GEMMs and the small index kernels of
    the host layer are not counted): per recurrent pass one attention plan, one opening norm and per
    layer rope_kv_write, attention + merge, SiLU-and-Mul and two sandwich norms; per draft offset one
    proposal kernel; acceptance (two launches), the round's uniforms when sampling, rollback."""
    passes = draft_loops * (k + 1) + target_loops - draft_loops
    per_pass = 2 + 6 * config.num_hidden_layers
    return passes * per_pass + k + 2 + (1 if sampled else 0) + 1


def copy_stats(stats):
    import copy

    return copy.copy(stats)


def attention_roofline(device, steps: int, warmup: int, parity_requests: int):
    """The verify attention at the kernel-microbench shape inside a 24-layer pass (KV write ->
    attention -> SiLU-and-Mul per layer, one plan per pass): CUDA-event time per attention call, its
    algorithmic bytes, and a comparison of layer 0's output for `parity_requests` requests with the
    CPU oracle.  Returns (roofline dict, parity dict, launches)."""
    import vllm_rlt_b200 as rlt

    work = Workload(seed=1234)
    g = torch.Generator(device=device).manual_seed(99)
    pool_shape = (work.total_pages, LAYERS, BLOCK, HEADS, HEAD_DIM)
    key_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
    value_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
    for pool in (key_pool, value_pool):  # N(0,1) * 0.5, generated in slabs to bound temporaries
        flat = pool.view(-1)
        slab = 1 << 28
        for start in range(0, flat.numel(), slab):
            n = min(slab, flat.numel() - start)
            flat[start:start + n] = (torch.randn(n, device=device, generator=g) * 0.5).to(torch.bfloat16)

    def mk(*shape, scale=1.0):
        return (torch.randn(*shape, device=device, generator=g) * scale).to(torch.bfloat16)

    q = mk(LAYERS, work.rows, HEADS, HEAD_DIM, scale=0.5)
    k_new = mk(LAYERS, work.kv_rows, HEADS, HEAD_DIM, scale=0.5)
    v_new = mk(LAYERS, work.kv_rows, HEADS, HEAD_DIM, scale=0.5)
    gate, up = mk(work.rows, FFN, scale=3.0), mk(work.rows, FFN)
    tables, lengths = work.tables.to(device), work.lengths.to(device)
    write_blocks, write_offsets = work.write_blocks.to(device), work.write_offsets.to(device)
    backend = rlt.create_backend(device, torch.bfloat16, HEAD_DIM, BLOCK)
    events, launches, first_out = [], 0, None
    for step in range(warmup + steps):
        with backend.kernel.shared_plan():
            for layer in range(LAYERS):
                kc, vc = key_pool[:, layer], value_pool[:, layer]
                rlt.kv_write(kc, vc, k_new[layer], v_new[layer], write_blocks, write_offsets)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                out = backend(q[layer], kc, vc, tables, lengths)
                b.record()
                rlt.silu_and_mul(gate, up)
                if step >= warmup:
                    events.append((a, b))
                    launches += 4
                if step == 0 and layer == 0:
                    first_out = out
        launches += 1 if step >= warmup else 0
    torch.cuda.synchronize()
    attention_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    status = backend.kernel.last_status(device)
    peak, peak_kind = measured_peaks()
    algorithmic = work.algorithmic_attention_bytes()
    achieved = algorithmic / (attention_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "verify_attention_kernel + merge_kernel, per layer call of a 24-layer pass "
                                          "(64 requests, ctx U[512,4096], 16 rows per request on a shared plane; "
                                          "inputs larger than L2: 34 GB pool streamed once per pass)",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "traffic": ATTENTION_TRAFFIC_RATIO * algorithmic,
                "traffic_source": "ncu dram bytes of a 32-request launch scaled by algorithmic bytes",
                "algorithmic_bytes": algorithmic, "avg_launch_ms": attention_ms, "timed_calls": len(events),
                "attention_status": status}
    parity = attention_parity(work, first_out, q[0], key_pool, value_pool, parity_requests)
    return roofline, parity, launches


def attention_parity(work, gpu_out, q0, key_pool, value_pool, requests: int):
    """Layer 0 of the full-size microbench against the CPU oracle for the first `requests` requests:
    their pages are copied to the host (with the new tokens' K/V already written), renumbered, and the
    oracle scores the same 16 rows per request.  Tolerance: 2e-2 absolute + 2e-2 relative (bf16)."""
    from oracle import oracle

    rows_per_request = TOKENS * DEPTHS
    pages = ((work.contexts + BLOCK - 1) // BLOCK)[:requests]
    ids = torch.cat([work.request_tables[i, : int(n)] for i, n in enumerate(pages.tolist())]).long()
    kc = key_pool[ids.to(key_pool.device), 0].cpu()
    vc = value_pool[ids.to(key_pool.device), 0].cpu()
    tables = torch.zeros(requests * rows_per_request, int(pages.max()), dtype=torch.int32)
    offset = 0
    for i, n in enumerate(pages.tolist()):
        tables[i * rows_per_request:(i + 1) * rows_per_request, :n] = torch.arange(offset, offset + n, dtype=torch.int32)
        offset += n
    rows = requests * rows_per_request
    want = oracle.paged_attention(q0[:rows].cpu(), kc, vc, tables, work.lengths[:rows]).float()
    got = gpu_out[:rows].float().cpu()
    diff = (got - want).abs()
    bound = 2e-2 + 2e-2 * want.abs()
    return {"against": "CPU oracle", "requests": requests, "rows": rows, "max_abs": float(diff.max()),
            "max_rel_of_bound": float((diff / bound).max()), "tolerance": "2e-2 abs + 2e-2 rel (bf16)",
            "ok": bool((diff <= bound).all())}


def run_gpu(args):
    import torch.distributed as dist

    import vllm_rlt_b200 as rlt

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- 1. the verify attention alone (roofline + parity), rank 0 ---------------------------
    roofline = parity = None
    attention_launches = 0
    if rank == 0:
        roofline, parity, attention_launches = attention_roofline(device, steps=min(args.steps, 10), warmup=2,
                                                                  parity_requests=4)
        gc.collect()
        torch.cuda.empty_cache()

    # ---- 2. self-speculative decoding: K rounds on the device clock, K on the host clock ------
    steps, warmup = args.steps, args.warmup
    k = DECODE_K
    e2e_warmup = min(warmup, 3)
    rounds_needed = warmup + steps + e2e_warmup + steps + 2
    max_tokens = max(DECODE_OUTPUT, rounds_needed * (k + 1))
    config = rlt.LoopedLMConfig()
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 3, device=device), device, torch.bfloat16)
    prompts = decode_prompts(DECODE_REQUESTS, DECODE_PROMPTS, config.vocab_size)
    decoder = rlt.SelfSpeculativeDecoder(model, cuda_graphs=True, capture_sizes=[DECODE_REQUESTS])
    torch.cuda.synchronize()
    t_open = time.perf_counter()
    session = decoder.open(prompts, max_tokens, num_speculative_tokens=k, draft_loops=DRAFT_LOOPS,
                           target_loops=TARGET_LOOPS, temperature=TEMPERATURE, seed=1, in_flight=2)
    torch.cuda.synchronize()
    open_seconds = time.perf_counter() - t_open
    stats = decoder.stats

    def run_rounds(count):
        """`count` rounds, two in flight, every one collected before this returns."""
        submitted = collected = 0
        while collected < count:
            while submitted < count and session.submit_round():
                submitted += 1
            if not session.collect_round():
                raise RuntimeError("the requests ran out of output budget inside the timed region")
            collected += 1

    run_rounds(warmup)
    barrier()
    clocks = ClockSampler(local)
    clocks.__enter__()
    before = copy_stats(stats)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    run_rounds(steps)
    stop.record()
    barrier()
    device_ms = start.elapsed_time(stop)
    after = copy_stats(stats)
    accepted = after.accepted_tokens - before.accepted_tokens
    committed = after.committed_tokens - before.committed_tokens
    drafted = after.drafted_tokens - before.drafted_tokens
    round_bytes = decode_round_bytes(config, before, after, steps, k)

    run_rounds(e2e_warmup)
    barrier()
    before_e2e = copy_stats(stats)
    t0 = time.perf_counter()
    run_rounds(steps)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    clocks.__exit__(None, None, None)
    after_e2e = copy_stats(stats)
    e2e_accepted = after_e2e.accepted_tokens - before_e2e.accepted_tokens
    runner = decoder.runner
    nb, w = runner.bucket_of(DECODE_REQUESTS), runner.width
    h2d, d2h = 3 * nb * 8, (nb * w + 4 * nb) * 8
    decode_status = model.attention.last_status(device)
    tokens_host = sum(len(r.generated_token_ids) for r in session.requests)

    times = torch.tensor([device_ms, e2e_ms, float(accepted), float(committed), float(e2e_accepted), float(drafted)],
                         dtype=torch.float64, device=device)
    table = times[None].cpu() if world == 1 else all_gather_rows(times)
    if rank == 0:
        per_step = table[:, :4].clone()
        per_step[:, 2:] /= steps                         # tokens of the timed window -> per step
        job = combine_ranks(per_step, world, steps)
        max_ms, mean_ms = float(table[:, 0].max()), float(table[:, 0].mean())
        e2e_value = float(table[:, 4].sum()) / (float(table[:, 1].max()) / 1e3)
        peak, peak_kind = measured_peaks()
        seconds = device_ms / 1e3
        per_round = launches_per_round(config, k, DRAFT_LOOPS, TARGET_LOOPS, True)
        line = {
            "metric": METRIC, "value": job["accepted_tokens_per_s"], "unit": "accepted tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": job["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": "configs[2]: Ouro-1.4B-shaped random-init bf16 model (24 layers, hidden 2048, 16x128 MHA, "
                            "FFN 5632, vocab 49152, 4 loops), 128 concurrent requests per GPU, prompts U[128,1024] of "
                            "uniform-random tokens, self-speculation k=4 from depth 2 verified at depth 4, rejection "
                            "sampling T=0.8; step = one speculative round of the whole batch (one CUDA graph), timed "
                            "in steady state after the prompt pass; roofline block: configs[1] verify attention",
                "requests_per_gpu": DECODE_REQUESTS, "k": k, "draft_loops": DRAFT_LOOPS, "target_loops": TARGET_LOOPS,
                "temperature": TEMPERATURE, "output_budget_tokens": max_tokens, "rounds_in_flight": 2,
                "kv_pool_gb": round(2 * session.runner.cache.key.numel() * 2 / 1e9, 2),
                "l2_policy": "inputs larger than L2 (every pass streams the active contexts' K/V and the layer weights)",
                "parallelism": f"{world} independent replicas decoding the same seeded requests, no collective",
                "prompt_pass_and_graph_capture_seconds": open_seconds,
            },
            "committed_tokens_per_s": job["committed_tokens_per_s"],
            "acceptance_rate": float(table[:, 2].sum()) / max(float(table[:, 5].sum()), 1.0),
            "accepted_per_step": job["accepted_per_step"], "committed_per_step": job["committed_per_step"],
            "rank_time_imbalance_max_over_mean": max_ms / mean_ms,
            "e2e": {"value": e2e_value, "unit": "accepted tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": float(table[:, 1].max()) / steps,
                    "path": "runner.submit(Python requests) -> graph replay -> ticket.collect() -> Python token lists, "
                            "host clock", "tokens_on_host": tokens_host},
            "gpu_launches": per_round * steps,
            "hbm_roofline_decode": {**round_bytes, "peak_gbs": peak, "peak_kind": peak_kind,
                                    "seconds_at_peak": round_bytes["total"] / (peak * 1e9),
                                    "frac": round_bytes["total"] / (peak * 1e9) / seconds},
            "roofline": roofline, "parity": parity,
            "clocks": clocks.summary(),
            "attention_status": decode_status,
        }
        if not args.no_cpu_baseline and world == 1:
            del session, decoder, model, runner
            gc.collect()
            torch.cuda.empty_cache()
            line["cpu_baseline"] = cpu_baseline(threads=os.cpu_count() or 1, rounds=2)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_attention_only(args):
    """Profiling aid: only the verify-attention calls of `--layers` layers for `--requests` requests
    (same shapes and seeds as the full step), timed per call with CUDA events.  Prints one JSON line."""
    import vllm_rlt_b200 as rlt

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    work = Workload(seed=1234, requests=args.requests, layers=args.layers, tokens=args.tokens, depths=args.depths,
                    context_range=(args.context_min, args.context_max),
                    kv_heads=args.kv_heads)
    g = torch.Generator(device=device).manual_seed(99)
    pool_shape = (work.total_pages, args.layers, BLOCK, args.kv_heads, HEAD_DIM)
    key_pool = (torch.randn(pool_shape, device=device, generator=g) * 0.5).to(torch.bfloat16)
    value_pool = (torch.randn(pool_shape, device=device, generator=g) * 0.5).to(torch.bfloat16)
    q = (torch.randn(args.layers, work.rows, HEADS, HEAD_DIM, device=device, generator=g) * 0.5).to(torch.bfloat16)
    tables, lengths = work.tables.to(device), work.lengths.to(device)
    backend = rlt.create_backend(device, torch.bfloat16, HEAD_DIM, BLOCK)
    events = []
    from contextlib import nullcontext
    for step in range(args.warmup + args.steps):
        with backend.kernel.shared_plan() if args.shared_plan else nullcontext():
            for layer in range(args.layers):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                backend(q[layer], key_pool[:, layer], value_pool[:, layer], tables, lengths)
                b.record()
                if step >= args.warmup:
                    events.append((a, b))
    torch.cuda.synchronize()
    ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    peak, kind = measured_peaks()
    algorithmic = work.algorithmic_attention_bytes()
    print(json.dumps({"only": "attention", "requests": args.requests, "layers": args.layers, "rows": work.rows,
                      "avg_call_ms": ms, "algorithmic_bytes": algorithmic,
                      "achieved_gbs": algorithmic / ms / 1e6, "frac": algorithmic / ms / 1e6 / peak,
                      "peak_kind": kind, "status": backend.kernel.last_status(device)}))


def run_prefill_only(args):
    """Profiling aid (`--only prefill`): packed causal prefill of `--requests` prompts of `--tokens`
    tokens each (16 x 128 MHA, bf16, 16-token pages, pages in random order) through
    `AttentionBackend.prefill`, timed per call with CUDA events.  Tensor-bound: reports TFLOP/s
    (4 * head_dim flops per visible (query, key) pair and head) against the measured bf16 peak."""
    import vllm_rlt_b200 as rlt

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    g = torch.Generator(device=device).manual_seed(17)
    n, seqs = args.tokens, args.requests
    pages = -(-n // BLOCK)
    total = pages * seqs
    shape = (total, 1, BLOCK, args.kv_heads, HEAD_DIM)
    both = (torch.randn((2,) + shape, device=device, generator=g) * 0.5).to(torch.bfloat16)
    key, value = both[0][:, 0], both[1][:, 0]
    tables = torch.randperm(total, device=device, generator=g).int().view(seqs, pages)
    lengths = torch.full((seqs,), n, dtype=torch.int32, device=device)
    cu = (torch.arange(seqs + 1, device=device) * n).int()
    q = (torch.randn(seqs * n, HEADS, HEAD_DIM, device=device, generator=g) * 0.5).to(torch.bfloat16)
    kernel = rlt.B200PagedAttention()
    max_new = n if not args.eager else 0          # --eager: the same rows through the grouped verify kernel
    for _ in range(args.warmup):
        kernel.prefill(q, key, value, tables, lengths, cu, max_new)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        kernel.prefill(q, key, value, tables, lengths, cu, max_new)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    flops = 4.0 * HEAD_DIM * HEADS * seqs * (n * (n + 1) / 2)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    print(json.dumps({"only": "prefill", "kernel": "grouped verify kernel" if args.eager else "prefill kernel",
                      "sequences": seqs, "tokens": n, "kv_heads": args.kv_heads, "ms_per_call": ms,
                      "algorithmic_flops": flops, "tflops": flops / ms / 1e9, "peak_tflops": peak,
                      "peak_kind": "measured" if peaks else "fallback", "frac": flops / ms / 1e9 / peak}))


def silu_comparison(device, steps: int, warmup: int):
    """SiLU-and-Mul at the path's shapes, this library's kernel beside the reference's own CUDA kernel when its
    extension (`vllm_rlt._C`, built from the reference's unmodified csrc for sm_100) is present under
    baseline/_ref: CUDA events, per call, L2-warm (the same tensors every call) and L2-cold (a ring of input
    sets larger than L2, so every call reads from HBM), plus one case where gate, up and out each start at a
    different 16-byte misalignment."""
    import glob

    import vllm_rlt_b200 as rlt

    kernels = {"b200": rlt.silu_and_mul}
    found = glob.glob(str(ROOT / "baseline" / "_ref" / "vllm_rlt" / "_C*.so"))
    note = None
    if found:
        try:
            torch.ops.load_library(found[0])
            kernels["reference"] = torch.ops.vllm_rlt.silu_and_mul
        except Exception as error:
            note = f"the reference extension did not load: {error}"
    else:
        note = "no reference extension under baseline/_ref"
    g = torch.Generator(device=device).manual_seed(3)
    peak, _ = measured_peaks()

    unroll = 32

    def timed(fn, sets):
        """Microseconds per call: a CUDA graph of `unroll` calls (as the reference's own benchmark of this
        kernel does, benchmarks/kernels/silu_and_mul.py there), replayed `steps` times, so that the host's
        per-call cost is not what is measured."""
        for i in range(max(warmup, 1)):
            fn(*sets[i % len(sets)])
        torch.cuda.synchronize()
        calls = max(unroll, len(sets))                 # every set of a cold ring is visited once per replay
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            kept = [fn(*sets[i % len(sets)]) for i in range(calls)]
        graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(max(steps, 1)):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        del kept
        return a.elapsed_time(b) / (max(steps, 1) * calls) * 1e3

    table = []
    for rows in (128, 640, 768, 1024):
        nbytes = 3 * rows * FFN * 2
        ring = max(2, int(400e6 // (2 * rows * FFN * 2)) + 1)            # inputs of the ring: > 3 x L2
        sets = [((torch.randn(rows, FFN, device=device, generator=g) * 3).to(torch.bfloat16),
                 torch.randn(rows, FFN, device=device, generator=g).to(torch.bfloat16)) for _ in range(ring)]
        row = {"shape": [rows, FFN], "dtype": "bf16", "bytes": nbytes}
        for name, fn in kernels.items():
            warm, cold = timed(fn, sets[:1]), timed(fn, sets)
            row[name] = {"warm_us": warm, "cold_us": cold, "cold_gbs": nbytes / cold / 1e3, "cold_frac": nbytes / cold / 1e3 / peak}
        if "reference" in kernels:
            assert torch.equal(kernels["b200"](*sets[0]), kernels["reference"](*sets[0]))
        table.append(row)
        del sets
    # independent misalignments: gate +2, up +4, (out is allocated by the op) elements off a 16-byte boundary
    rows = 640
    base = [torch.randn(rows * FFN + 16, device=device, generator=g).to(torch.bfloat16) for _ in range(2)]
    gate, up = base[0][1:1 + rows * FFN].view(rows, FFN), base[1][2:2 + rows * FFN].view(rows, FFN)
    row = {"shape": [rows, FFN], "dtype": "bf16", "misaligned": "gate +2 bytes, up +4 bytes", "bytes": 3 * rows * FFN * 2}
    for name, fn in kernels.items():
        row[name] = {"warm_us": timed(fn, [(gate, up)])}
    table.append(row)
    return {"silu_and_mul": table, "reference_kernel": "vllm_rlt._C built from the reference's csrc for sm_100"
            if "reference" in kernels else None, "note": note}


def run_small_only(args):
    """Profiling aid: the acceptance kernels (`--only accept`) or SiLU-and-Mul (`--only silu`) at the
    step's shapes, a few hundred MB on the device, timed per call with CUDA events."""
    import vllm_rlt_b200 as rlt

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    work = Workload(seed=1234, requests=args.requests, layers=1)
    out = {"only": args.only, "requests": args.requests}

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    if args.only == "silu":
        out.update(silu_comparison(device, args.steps, args.warmup))
    else:
        x = {k: v.to(device) for k, v in work.host_inputs(pin=False).items() if k not in ("q", "k", "v", "gate", "up")}
        per_row_t = x["temperature"].repeat_interleave(TOKENS)
        slot_values = torch.zeros(2 * work.requests, 2, dtype=torch.int64, device=device)
        drafts, _ = rlt.sample_rows(x["draft"], per_row_t, x["u_draft"])
        tokens = torch.zeros(work.requests, TOKENS, dtype=torch.int64, device=device)
        tokens[:, 1:] = drafts.view(work.requests, TOKENS)[:, :-1]
        logits_bytes = x["target"].numel() * 4
        out["sample_rows_ms"] = timed(lambda: rlt.sample_rows(x["draft"], per_row_t, x["u_draft"]))
        out["accept_greedy_ms"] = timed(lambda: rlt.accept_greedy(x["target"], x["cu_rows"], tokens, x["starts"],
                                                                  x["slots"], slot_values))
        out["accept_rejection_ms"] = timed(lambda: rlt.accept_rejection(
            x["target"], x["draft"], x["cu_rows"], tokens, x["starts"], x["temperature"], x["u_accept"],
            x["u_final"], x["slots"], slot_values))
        result, _ = rlt.accept_rejection(x["target"], x["draft"], x["cu_rows"], tokens, x["starts"],
                                         x["temperature"], x["u_accept"], x["u_final"])
        accepted = result[work.accept_rows:work.accept_rows + work.requests]
        out["rollback_ms"] = timed(lambda: rlt.rollback(x["starts"], accepted + 1, x["request_tables"], BLOCK))
        # the same draws and acceptance with top-k = 50 / top-p = 0.9 on every request (radix-select cut)
        n = work.requests
        top_k, top_p = torch.full((n,), 50, dtype=torch.int32, device=device), torch.full((n,), 0.9, device=device)
        row_k, row_p = top_k.repeat_interleave(TOKENS), top_p.repeat_interleave(TOKENS)
        out["sample_rows_top_k_top_p_ms"] = timed(lambda: rlt.sample_rows(x["draft"], per_row_t, x["u_draft"], row_k, row_p))
        out["accept_rejection_top_k_top_p_ms"] = timed(lambda: rlt.accept_rejection(
            x["target"], x["draft"], x["cu_rows"], tokens, x["starts"], x["temperature"], x["u_accept"], x["u_final"],
            top_k=top_k, top_p=top_p))
        out["probabilities_top_p_ms"] = timed(lambda: rlt.probabilities(x["target"], per_row_t, None, row_p))
        out.update(rows=work.accept_rows, vocab=VOCAB, greedy_bytes=logits_bytes, rejection_bytes=2 * logits_bytes,
                   greedy_gbs=logits_bytes / out["accept_greedy_ms"] / 1e6,
                   rejection_gbs=2 * logits_bytes / out["accept_rejection_ms"] / 1e6)
    print(json.dumps(out))


def run_decode_workload(args):
    """Secondary workload (`--workload decode`): self-speculative decoding of a random-init
    Ouro-1.4B-shaped model (24 layers, hidden 2048, 16 x 128 MHA, FFN 5632, vocab 49152, 4 loops, bf16)
    through `vllm_rlt_b200.SelfSpeculativeDecoder` — the bench line's workload run to completion, with the output length set by
    `--output-tokens`.  The GEMMs are cuBLAS; every recurrent loop is replayed from a CUDA graph per
    row bucket unless `--eager` is given.  The prefill and the graph captures are outside the timed region."""
    import vllm_rlt_b200 as rlt

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    config = rlt.LoopedLMConfig()
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 3, device=device), device, torch.bfloat16)
    g = torch.Generator().manual_seed(11)
    lengths = torch.randint(args.prompt_min, args.prompt_max + 1, (args.requests,), generator=g).tolist()
    prompts = [torch.randint(1, config.vocab_size, (n,), generator=g).tolist() for n in lengths]
    if args.shared_prefix > 0:   # every second request starts with one common prefix (a long-context mix with shared prefixes)
        common = torch.randint(1, config.vocab_size, (args.shared_prefix,), generator=g).tolist()
        prompts = [common[:len(p) - 1] + p[len(common[:len(p) - 1]):] if i % 2 else p for i, p in enumerate(prompts)]
    decoder = rlt.SelfSpeculativeDecoder(model, cuda_graphs=not args.eager, prefix_caching=args.prefix_caching,
                                         capture_sizes=sorted({args.requests, max(args.requests // 2, 1),
                                                               max(args.requests // 4, 1)}))
    clock = {}

    def start_clock():
        torch.cuda.synchronize()
        clock["start"] = time.perf_counter()

    torch.cuda.synchronize()
    clock["begin"] = time.perf_counter()
    tokens = decoder.generate(prompts, args.output_tokens, num_speculative_tokens=args.k, draft_loops=DRAFT_LOOPS,
                              target_loops=TARGET_LOOPS, temperature=args.temperature, seed=1, after_prefill=start_clock,
                              in_flight=args.in_flight)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - clock["start"]
    stats = decoder.stats
    # HBM roofline of the decode loop: every recurrent pass streams the layer weights once and the
    # K/V of every active request's context once per layer; every LM-head call streams lm_head once
    # (counted per draft pass and per round).  Activations and logits are left out (a few percent).
    c = config
    layer_params = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                    + c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    weight_bytes = 2.0 * c.num_hidden_layers * layer_params * stats.loop_passes
    kv_bytes = 2.0 * 2 * c.num_key_value_heads * c.head_dim * c.num_hidden_layers * stats.context_tokens_read
    head_calls = stats.rounds / max(args.requests, 1) * (args.k + 1)   # upper bound: k draft calls + 1 verify call per round
    head_bytes = 2.0 * c.vocab_size * c.hidden_size * head_calls
    peak, peak_kind = measured_peaks()
    roofline_s = (weight_bytes + kv_bytes + head_bytes) / (peak * 1e9)
    print(json.dumps({
        "workload": f"decode: Ouro-1.4B-shaped random-init bf16, self-spec k={args.k} from depth 2, "
                    f"{args.requests} requests, prompts U[{args.prompt_min},{args.prompt_max}]"
                    + (f" (every second one behind a common {args.shared_prefix}-token prefix, prefix reuse "
                       f"{'on' if args.prefix_caching else 'off'})" if args.shared_prefix else "")
                    + f", {args.output_tokens} output tokens, T={args.temperature}, "
                    + ("eager launches" if args.eager else "every round one CUDA graph") + f", {args.in_flight} round(s) in flight",
        "total_seconds": time.perf_counter() - clock["begin"],
        "prefill_and_capture_seconds": clock["start"] - clock["begin"], "prompt_tokens": sum(lengths),
        "prompt_tokens_computed": stats.prompt_tokens_computed, "prefix_hit_tokens": stats.prefix_hit_tokens,
        "decode_seconds": seconds, "committed_tokens": stats.committed_tokens, "accepted_tokens": stats.accepted_tokens,
        "drafted_tokens": stats.drafted_tokens, "request_rounds": stats.rounds,
        "committed_tokens_per_s": stats.committed_tokens / seconds,
        "accepted_tokens_per_s": stats.accepted_tokens / seconds,
        "acceptance_rate": stats.accepted_tokens / max(stats.drafted_tokens, 1),
        "loop_passes": stats.loop_passes,
        "hbm_roofline": {"kv_bytes": kv_bytes, "weight_bytes": weight_bytes, "lm_head_bytes": head_bytes,
                         "peak_gbs": peak, "peak_kind": peak_kind, "seconds_at_peak": roofline_s,
                         "frac": roofline_s / seconds},
        "tokens_out": sum(len(t) for t in tokens), "attention_status": model.attention.last_status(device)}))


def run_reference_engine_workload(args):
    """`--workload decode --engine reference`: the decode workload's requests through the unmodified vllm-rlt
    engine on the GPU (an installed copy under baseline/_ref; nothing of this library on the path): the model
    class of the reference with the same seeded weights, its scheduler and speculative runner, its Triton paged
    attention, its CUDA graphs.  Timing follows the reference's own benchmark: the decode clock starts when
    every request has its first token and the device is idle, counts the tokens produced from then on and
    stops after the device has finished."""
    import vllm_rlt_b200 as rlt

    reference_root = ROOT / "baseline" / "_ref"
    if not (reference_root / "vllm_rlt").is_dir():
        print(json.dumps({"engine": "reference", "unavailable": "no copy of the reference under baseline/_ref"}))
        return
    sys.path.insert(0, str(reference_root))
    from vllm_rlt import CacheConfig, ExecutionConfig, SamplingParams, SpeculativeConfig
    from vllm_rlt.config import SchedulerConfig
    from vllm_rlt.engine.stage_engine import StageEngine
    from vllm_rlt.models import OuroConfig, OuroForCausalLM

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    ours = rlt.LoopedLMConfig()
    shape = {name: getattr(ours, name) for name in (
        "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
        "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "total_ut_steps")}
    config = OuroConfig(**shape, max_position_embeddings=4096, bos_token_id=0, eos_token_id=0)
    with torch.device(device):
        model = OuroForCausalLM(config).to(torch.bfloat16)
    state = rlt.seeded_state_dict(ours, 3, device=device)
    model.load_state_dict({name: state[name] for name in model.state_dict()}, strict=True)
    del state
    prompts = decode_prompts(args.requests, (args.prompt_min, args.prompt_max), config.vocab_size)
    pages = sum(-(-(len(p) + args.output_tokens + args.k + 2) // BLOCK) for p in prompts) * config.total_ut_steps + 64
    if args.adopt != "nothing":
        # What a maintainer of the reference adds to adopt the kernels: one more backend name that wraps
        # B200PagedAttention in the reference's own AttentionBackend / BackendCapabilities classes.
        import dataclasses

        from vllm_rlt.attention import backend as backend_module
        from vllm_rlt.core import kv_cache_manager as cache_module

        validate, create = backend_module.validate_backend_name, backend_module._create_explicit

        def explicit(name, device_, dtype, head_dim, block_size):
            if name != "b200":
                return create(name, device_, dtype, head_dim, block_size)
            native = rlt.create_backend(device_, dtype, head_dim, block_size)
            capabilities = backend_module.BackendCapabilities(**dataclasses.asdict(native.capabilities))
            return backend_module.AttentionBackend(native.kernel, capabilities, {"backend": "b200"})

        backend_module.validate_backend_name = cache_module.validate_backend_name = \
            lambda name: None if name == "b200" else validate(name)
        backend_module._create_explicit = explicit
        rlt.register_torch_op("vllm_rlt")
    engine = StageEngine(
        model, cache_config=CacheConfig(pages, BLOCK), attention_backend="triton" if args.adopt == "nothing" else "b200",
        scheduler_config=SchedulerConfig(max_num_seqs=args.requests,
                                         max_num_batched_tokens=max(2048, args.requests * (args.k + 1))),
        execution_config=ExecutionConfig(async_scheduling=not args.sync, cuda_graphs=not args.eager),
        speculative_config=SpeculativeConfig(args.k, draft_loops=DRAFT_LOOPS, target_loops=TARGET_LOOPS))
    if args.adopt == "runner":
        # ... and the runner: this library's looped LM over the reference's weights and KV-cache manager, in the place of
        # the engine's own speculative runner (device-resident protocol under the async engine, synchronous otherwise).
        native_model = rlt.LoopedLM(ours, model.state_dict(), device, torch.bfloat16)
        view = rlt.KVCacheManagerView(engine.cache_manager, max_pages=-(-config.max_position_embeddings // BLOCK))
        runner = rlt.B200SpeculativeRunner(
            native_model, view, rlt.SpeculativeConfig(args.k, draft_loops=DRAFT_LOOPS, target_loops=TARGET_LOOPS),
            max_num_seqs=args.requests, cuda_graphs=not args.eager, capture_sizes=[args.requests],
            compute_stream=engine.model_runner.core_stream, report_frontiers=not args.sync)
        engine.speculative_runner = engine.executor.speculation = runner
    params = SamplingParams(max_tokens=args.output_tokens, ignore_eos=True, temperature=args.temperature, seed=1)
    torch.cuda.synchronize()
    begin = time.perf_counter()
    for i, prompt in enumerate(prompts):
        engine.add_request(str(i), prompt, params)
    produced, finished, start, at_start = {}, 0, None, 0
    while engine.has_unfinished_requests():
        for output in engine.step():
            produced[output.request_id] = len(output.token_ids)
            finished += bool(output.finished)
        if start is None and len(produced) == args.requests:
            torch.cuda.synchronize()
            start, at_start = time.perf_counter(), sum(produced.values())
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start
    stats = engine.speculative_runner.stats
    print(json.dumps({
        "engine": "vllm-rlt reference on the GPU, " + {"nothing": "unmodified", "attention": "with this library's attention "
                  "backend and SiLU op", "runner": "with this library's attention backend and speculative runner"}[args.adopt],
        "attention_backend": "triton" if args.adopt == "nothing" else "b200",
        "async_scheduling": not args.sync, "cuda_graphs": not args.eager,
        "workload": f"decode: Ouro-1.4B-shaped random-init bf16, self-spec k={args.k} from depth 2, {args.requests} requests, "
                    f"prompts U[{args.prompt_min},{args.prompt_max}], {args.output_tokens} output tokens, T={args.temperature}",
        "total_seconds": time.perf_counter() - begin, "prompt_pass_seconds": start - begin, "decode_seconds": seconds,
        "decode_tokens": sum(produced.values()) - at_start,
        "decode_tokens_per_s": (sum(produced.values()) - at_start) / seconds,
        "accepted_tokens": stats.accepted_tokens, "drafted_tokens": stats.drafted_tokens, "request_rounds": stats.rounds,
        "accepted_tokens_per_s_over_the_whole_run": stats.accepted_tokens / (time.perf_counter() - begin),
        "finished_requests": finished}))


def balanced_shards(lengths, world: int):
    """Longest-first greedy assignment of requests to ranks by prompt length: returns one list of request
    indices per rank whose total lengths differ by at most one request's length."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    loads, shards = [0] * world, [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda x: (loads[x], len(shards[x])))
        shards[r].append(i)
        loads[r] += lengths[i]
    return shards


def waves_under_budget(indices, lengths, tokens_extra: int, bytes_per_token: int, budget_bytes: float, max_wave: int):
    """Consecutive groups of a rank's requests whose reserved KV (prompt + output + drafts, every depth
    plane) fits the budget, at most `max_wave` requests each."""
    waves, current, used = [], [], 0.0
    for i in indices:
        need = (lengths[i] + tokens_extra) * bytes_per_token
        if current and (used + need > budget_bytes or len(current) >= max_wave):
            waves.append(current)
            current, used = [], 0.0
        current.append(i)
        used += need
    if current:
        waves.append(current)
    return waves


def run_sharded_workload(args):
    """`--workload sharded`: a fixed set of requests (default 1024, prompts U[256, 2048], 512 output tokens,
    k = 6, rejection sampling at T = 0.8) shared out over the ranks by prompt length and decoded to completion by every rank's own
    engine in waves that fit its KV pool — whole-job strong scaling, prompt passes and graph captures
    included.  One rank per GPU, no collective on the path; the job's time is the slowest rank's."""
    import torch.distributed as dist

    import vllm_rlt_b200 as rlt

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    config = rlt.LoopedLMConfig(num_hidden_layers=args.model_layers)
    model = rlt.LoopedLM(config, rlt.seeded_state_dict(config, 3, device=device), device, torch.bfloat16)
    prompts = decode_prompts(args.total_requests, (args.prompt_min, args.prompt_max), config.vocab_size, seed=23)
    if args.shared_prefix > 0:   # every second request starts with one common prefix
        common = decode_prompts(1, (args.shared_prefix, args.shared_prefix), config.vocab_size, seed=29)[0]
        prompts = [common[:len(p) - 1] + p[len(common[:len(p) - 1]):] if i % 2 else p for i, p in enumerate(prompts)]
    lengths = [len(p) for p in prompts]
    mine = balanced_shards(lengths, world)[rank]
    bytes_per_token = (config.total_ut_steps * config.num_hidden_layers * 2 * config.num_key_value_heads
                       * config.head_dim * 2)
    waves = waves_under_budget(mine, lengths, args.output_tokens + args.k + 1 + BLOCK, bytes_per_token,
                               args.kv_budget_gb * 1e9, args.max_wave)
    # The engine's fixed resources, built once: a pool that holds the largest wave, one runner over it and
    # the round graphs of three batch sizes.  A wave gets the pool's pages afresh; nothing is re-captured.
    extra = args.output_tokens + args.k + 1
    pages_of = lambda i: -(-(lengths[i] + extra) // BLOCK)
    pool_pages = max(sum(pages_of(i) for i in wave) for wave in waves) * config.total_ut_steps
    largest = max(len(wave) for wave in waves)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    kv = rlt.PagedKV.reserve(model, pool_pages, largest, max(pages_of(i) for i in mine), BLOCK)
    runner = rlt.B200SpeculativeRunner(model, kv, rlt.SpeculativeConfig(args.k, DRAFT_LOOPS, TARGET_LOOPS),
                                       max_num_seqs=largest, cuda_graphs=not args.eager,
                                       capture_sizes=sorted({largest, max(largest // 2, 1), max(largest // 4, 1)}))
    accepted = committed = drafted = rounds = prefix_hits = 0
    for wave in waves:
        decoder = rlt.SelfSpeculativeDecoder(model, cuda_graphs=not args.eager, prefix_caching=args.prefix_caching)
        session = decoder.open([prompts[i] for i in wave], args.output_tokens, num_speculative_tokens=args.k,
                               draft_loops=DRAFT_LOOPS, target_loops=TARGET_LOOPS, temperature=args.temperature, seed=1,
                               in_flight=args.in_flight, kv=kv, runner=runner)
        before = (runner.stats.drafted_tokens, runner.stats.rounds)
        session.run()
        session.close()
        s = decoder.stats
        accepted, committed = accepted + s.accepted_tokens, committed + s.committed_tokens
        drafted += runner.stats.drafted_tokens - before[0]
        rounds += s.loop_passes
        prefix_hits += s.prefix_hit_tokens
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    row = torch.tensor([seconds, float(accepted), float(committed), float(drafted), float(len(mine)),
                        float(sum(lengths[i] for i in mine)), float(len(waves)), float(prefix_hits)],
                       dtype=torch.float64, device=device)
    table = row[None].cpu() if world == 1 else all_gather_rows(row)
    if rank == 0:
        slowest, mean = float(table[:, 0].max()), float(table[:, 0].mean())
        print(json.dumps({
            "workload": f"sharded: {args.total_requests} requests in total, prompts U[{args.prompt_min},{args.prompt_max}], "
                        f"{args.output_tokens} output tokens, k={args.k}, T={args.temperature}, LAST_EXITED planes, every "
                        f"request verified at depth {TARGET_LOOPS}; length-balanced over {world} rank(s), waves of at most "
                        f"{args.max_wave} requests within {args.kv_budget_gb} GB of KV",
            "n_gpus": world, "scaling": "strong", "job_seconds": slowest,
            "rank_time_imbalance_max_over_mean": slowest / mean,
            "accepted_tokens_per_s": float(table[:, 1].sum()) / slowest,
            "committed_tokens_per_s": float(table[:, 2].sum()) / slowest,
            "acceptance_rate": float(table[:, 1].sum()) / max(float(table[:, 3].sum()), 1.0),
            "model_layers": args.model_layers, "shared_prefix_tokens": args.shared_prefix,
            "prefix_caching": bool(args.prefix_caching), "prompt_tokens_mapped_from_the_prefix_index": float(table[:, 7].sum()),
            "requests_per_rank": table[:, 4].tolist(), "prompt_tokens_per_rank": table[:, 5].tolist(),
            "waves_per_rank": table[:, 6].tolist(), "seconds_per_rank": table[:, 0].tolist()}))
    if world > 1:
        dist.destroy_process_group()


class CpuDecodeSample:
    """The decode round of the bench on the host cores: the reference's Torch path for a speculative
    round (worker/speculative.py:418-511 of the reference) restated over the CPU oracle's kernels
    (paged attention, KV write, SiLU-and-Mul, sampler, rejection acceptance) and torch CPU GEMMs, bf16.

    A bounded sample: `sample` of the 128 requests carry real contexts (attention, KV write, sampling
    and acceptance run for them and are scaled by 128 / sample); the GEMMs, whose cost on a CPU is set
    by the weights they stream rather than by a handful of rows, run at the FULL batch's row counts (128
    rows per draft pass, 640 per verify pass, zero rows as filler) and are not scaled.  The prompts are
    not run on the CPU (minutes): the sampled requests' pages hold seeded random K/V of the contexts'
    lengths, which costs the same to attend to."""

    def __init__(self, threads: int, sample: int = 8):
        from oracle import oracle
        from vllm_rlt_b200.looped_lm import LoopedLMConfig, rms_norm, rotate_half, seeded_state_dict

        torch.set_num_threads(threads)
        os.environ.setdefault("OMP_NUM_THREADS", str(threads))
        self.oracle, self.rms_norm, self.rotate_half = oracle, rms_norm, rotate_half
        self.config = c = LoopedLMConfig()
        self.sample, self.k = sample, DECODE_K
        self.w = {n: t.to(torch.bfloat16) for n, t in seeded_state_dict(c, 3).items()}
        g = torch.Generator().manual_seed(11)
        prompts = torch.randint(DECODE_PROMPTS[0], DECODE_PROMPTS[1] + 1, (DECODE_REQUESTS,), generator=g)[:sample]
        self.starts = prompts + DECODE_OUTPUT // 2                      # mid-generation positions
        width = self.k + 1
        pages = (self.starts + width + BLOCK) // BLOCK
        planes = c.total_ut_steps
        total = int(pages.sum()) * planes
        order = torch.randperm(total, generator=g).int()
        self.tables = torch.zeros(sample, planes, int(pages.max()), dtype=torch.int32)
        cursor = 0
        for i, n in enumerate(pages.tolist()):
            for p in range(planes):
                self.tables[i, p, :n] = order[cursor:cursor + n]
                cursor += n
        shape = (total, c.num_hidden_layers, BLOCK, c.num_key_value_heads, c.head_dim)
        seed_block = (torch.randn(1 << 24, generator=g) * 0.5).to(torch.bfloat16)
        self.key, self.value = torch.empty(shape, dtype=torch.bfloat16), torch.empty(shape, dtype=torch.bfloat16)
        for pool, shift in ((self.key, 0), (self.value, 7919)):
            flat = pool.view(-1)
            for start in range(0, flat.numel(), seed_block.numel()):
                n = min(seed_block.numel(), flat.numel() - start)
                flat[start:start + n] = seed_block.roll(shift)[:n]
        self.tokens0 = torch.randint(1, c.vocab_size, (sample,), generator=g)
        self.inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
        self.generator = g
        self.gemm_s = self.other_s = 0.0

    def linear(self, x, weight, full_rows):
        padded = torch.zeros(full_rows, x.shape[1], dtype=x.dtype)
        padded[: x.shape[0]] = x
        t = time.perf_counter()
        y = torch.nn.functional.linear(padded, weight)
        self.gemm_s += time.perf_counter() - t
        return y[: x.shape[0]]

    def loop(self, hidden, positions, request_of_row, plane, full_rows):
        """One recurrent loop over all layers (models/ouro.py:171-221, 283-291 of the reference)."""
        c, w, o = self.config, self.w, self.oracle
        rows = hidden.shape[0]
        angles = positions.float().unsqueeze(-1) * self.inv_freq
        angles = torch.cat((angles, angles), -1)
        cos, sin = angles.cos().to(torch.bfloat16).unsqueeze(1), angles.sin().to(torch.bfloat16).unsqueeze(1)
        tables = self.tables[request_of_row, plane].contiguous()
        blocks = tables.gather(1, (positions // BLOCK)[:, None]).squeeze(1).long()
        offsets, lengths = positions % BLOCK, (positions + 1).int()
        for layer in range(c.num_hidden_layers):
            p = f"model.layers.{layer}."
            x = self.rms_norm(hidden, w[p + "input_layernorm.weight"], c.rms_norm_eps)
            q = self.linear(x, w[p + "self_attn.q_proj.weight"], full_rows).view(rows, -1, c.head_dim)
            k = self.linear(x, w[p + "self_attn.k_proj.weight"], full_rows).view(rows, -1, c.head_dim)
            v = self.linear(x, w[p + "self_attn.v_proj.weight"], full_rows).view(rows, -1, c.head_dim)
            q = q * cos + self.rotate_half(q) * sin
            k = k * cos + self.rotate_half(k) * sin
            kc, vc = self.key[:, layer], self.value[:, layer]
            o.kv_write(kc, vc, k.contiguous(), v.contiguous(), blocks, offsets)
            attended = o.paged_attention(q.contiguous(), kc, vc, tables, lengths).reshape(rows, -1)
            attended = self.linear(attended, w[p + "self_attn.o_proj.weight"], full_rows)
            hidden = hidden + self.rms_norm(attended, w[p + "input_layernorm_2.weight"], c.rms_norm_eps)
            x = self.rms_norm(hidden, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            gate = self.linear(x, w[p + "mlp.gate_proj.weight"], full_rows)
            up = self.linear(x, w[p + "mlp.up_proj.weight"], full_rows)
            mlp = self.linear(o.silu_and_mul(gate.contiguous(), up.contiguous()), w[p + "mlp.down_proj.weight"], full_rows)
            hidden = hidden + self.rms_norm(mlp, w[p + "post_attention_layernorm_2.weight"], c.rms_norm_eps)
        return self.rms_norm(hidden, w["model.norm.weight"], c.rms_norm_eps)

    def round(self):
        """One speculative round of the sampled requests; returns accepted tokens of the sample."""
        c, o, n, width = self.config, self.oracle, self.sample, self.k + 1
        g = self.generator
        begin, gemm_before = time.perf_counter(), self.gemm_s
        temperature = torch.full((n,), TEMPERATURE)
        tokens = torch.zeros(n, width, dtype=torch.int64)
        tokens[:, 0] = self.tokens0
        requests = torch.arange(n)
        retained, draft_logits = [], torch.zeros(n * width, c.vocab_size, dtype=torch.bfloat16)
        for offset in range(width):
            hidden = torch.nn.functional.embedding(tokens[:, offset], self.w["model.embed_tokens.weight"])
            for depth in range(DRAFT_LOOPS):
                hidden = self.loop(hidden, self.starts + offset, requests, depth, DECODE_REQUESTS)
            retained.append(hidden)
            if offset + 1 == width:
                break
            logits = self.linear(hidden, self.w["lm_head.weight"], DECODE_REQUESTS)
            draft_logits.view(n, width, -1)[:, offset] = logits
            proposed, _ = o.sample_rows(logits.contiguous(), temperature, torch.rand(n, generator=g))
            tokens[:, offset + 1] = proposed.clamp_min(0)
        hidden = torch.stack(retained, 1).reshape(n * width, -1)
        row_request = requests.repeat_interleave(width)
        positions = (self.starts[:, None] + torch.arange(width)[None, :]).reshape(-1)
        for depth in range(DRAFT_LOOPS, TARGET_LOOPS):
            hidden = self.loop(hidden, positions, row_request, depth, DECODE_REQUESTS * width)
        logits = self.linear(hidden, self.w["lm_head.weight"], DECODE_REQUESTS * width).contiguous()
        cu = (torch.arange(n + 1) * width).int()
        result, _ = o.accept_rejection(logits, draft_logits, cu, tokens, self.starts.clone(), temperature,
                                       torch.rand(n * width, generator=g), torch.rand(n, generator=g))
        accepted = result[n * width: n * width + n]
        o.rollback(self.starts.clone(), accepted + 1, self.tables, BLOCK)
        total = time.perf_counter() - begin
        self.other_s += total - (self.gemm_s - gemm_before)
        return int(accepted.sum())


def cpu_decode_rounds(threads: int, rounds: int, warmup: int = 1, sample: int = 8):
    """Times `rounds` CPU rounds of the bounded sample; returns the estimate for the full batch."""
    cpu = CpuDecodeSample(threads, sample)
    for _ in range(warmup):
        cpu.round()
    cpu.gemm_s = cpu.other_s = 0.0
    accepted = sum(cpu.round() for _ in range(rounds))
    scale = DECODE_REQUESTS / sample
    round_s = (cpu.gemm_s + scale * cpu.other_s) / rounds
    accepted_per_round = scale * accepted / rounds
    text = (f"{sample} of {DECODE_REQUESTS} requests x {rounds} rounds (k={DECODE_K}, T={TEMPERATURE}): attention, KV write, "
            f"sampler and acceptance for the sampled requests {cpu.other_s:.1f} s, scaled x{scale:.0f}; GEMMs at the full "
            f"batch's row counts {cpu.gemm_s:.1f} s, not scaled; prompts not run on the CPU (seeded random K/V)")
    return {"round_s": round_s, "accepted_per_round": accepted_per_round, "sample": text,
            "cores": cpu.oracle.num_threads(), "measured_s": cpu.gemm_s + cpu.other_s}


def cpu_baseline(threads: int, rounds: int):
    r = cpu_decode_rounds(threads, rounds)
    return {"value": r["accepted_per_round"] / r["round_s"], "unit": "accepted tokens/s", "cores": r["cores"],
            "kind": "port", "sample": r["sample"], "estimated_s_per_step": r["round_s"]}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's Torch path for the same speculative
    rounds (the reference package is Python over PyTorch and is not present where the bench runs),
    timed on all host cores; each step is the bounded sample described in `CpuDecodeSample`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    r = cpu_decode_rounds(threads, steps, warmup)
    value = r["accepted_per_round"] / r["round_s"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "accepted tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": warmup,
        "ms_per_step": r["round_s"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[2] speculative rounds on the host cores (CPU port of the reference's Torch path, "
                               "bounded sample scaled to the full batch of 128 requests)"},
        "cpu_baseline": {"value": value, "unit": "accepted tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": value, "unit": "accepted tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--only", default=None, choices=["attention", "accept", "silu", "prefill"],
                        help="profiling aid: run only this kernel family (not a bench line)")
    parser.add_argument("--workload", default="rounds", choices=["rounds", "decode", "sharded"],
                        help="rounds: timed speculative rounds (the bench line); decode: one complete generation; "
                             "sharded: a fixed request set shared out over the ranks, decoded to completion")
    parser.add_argument("--engine", default="b200", choices=["b200", "reference"],
                        help="decode workload: this library's decoder, or the unmodified reference engine on the GPU")
    parser.add_argument("--sync", action="store_true", help="decode workload, reference engine: its synchronous runner")
    parser.add_argument("--adopt", default="nothing", choices=["nothing", "attention", "runner"],
                        help="decode workload, reference engine: what of this library the engine adopts (nothing: the "
                             "unmodified reference; attention: the b200 attention backend and SiLU op; runner: also the "
                             "speculative runner)")
    parser.add_argument("--k", type=int, default=None, help="decode / sharded workloads: drafts per round")
    parser.add_argument("--in-flight", type=int, default=2, help="decode / sharded workloads: rounds in flight (1 or 2)")
    parser.add_argument("--total-requests", type=int, default=1024, help="sharded workload: requests over all ranks")
    parser.add_argument("--kv-budget-gb", type=float, default=140.0, help="sharded workload: KV bytes a wave may reserve")
    parser.add_argument("--max-wave", type=int, default=128, help="sharded workload: most requests decoded together")
    parser.add_argument("--model-layers", type=int, default=LAYERS, help="sharded workload: decoder layers of the model (24; 48 for the 2.6B shape)")
    parser.add_argument("--output-tokens", type=int, default=None,
                        help="decode workload: tokens per request (default 32); sharded workload: default 512")
    parser.add_argument("--eager", action="store_true", help="decode workload: launch every kernel from the host")
    parser.add_argument("--prompt-min", type=int, default=None, help="shortest prompt (decode: 128, sharded: 256)")
    parser.add_argument("--prompt-max", type=int, default=None, help="longest prompt (decode: 1024, sharded: 2048)")
    parser.add_argument("--shared-prefix", type=int, default=0,
                        help="decode / sharded workloads: every second prompt starts with one common prefix of this many tokens")
    parser.add_argument("--prefix-caching", action="store_true", help="decode / sharded workloads: map shared prompt pages instead of recomputing them")
    parser.add_argument("--temperature", type=float, default=None,
                        help="sampling temperature (default 0.8; 0 = greedy)")
    parser.add_argument("--requests", type=int, default=REQUESTS)
    parser.add_argument("--layers", type=int, default=LAYERS)
    parser.add_argument("--tokens", type=int, default=TOKENS, help="with --only attention: new tokens per request")
    parser.add_argument("--depths", type=int, default=DEPTHS, help="with --only attention: depth rows per token")
    parser.add_argument("--context-min", type=int, default=512, help="with --only attention: shortest context")
    parser.add_argument("--context-max", type=int, default=4096, help="with --only attention: longest context")
    parser.add_argument("--kv-heads", type=int, default=HEADS, help="with --only attention: KV heads (query heads stay 16)")
    parser.add_argument("--shared-plan", action="store_true",
                        help="with --only attention: plan once per pass instead of once per layer call")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the verify-step kernels have no CPU fallback")
    sharded = args.workload == "sharded"
    for name, decode_default, sharded_default in (("k", DECODE_K, 6), ("output_tokens", 32, 512), ("prompt_min", 128, 256),
                                                  ("prompt_max", 1024, 2048), ("temperature", TEMPERATURE, TEMPERATURE)):
        if getattr(args, name) is None:
            setattr(args, name, sharded_default if sharded else decode_default)
    if sharded:
        run_sharded_workload(args)
        return
    if args.workload == "decode":
        if args.engine == "reference":
            run_reference_engine_workload(args)
        else:
            run_decode_workload(args)
        return
    if args.only == "attention":
        run_attention_only(args)
        return
    if args.only == "prefill":
        run_prefill_only(args)
        return
    if args.only in ("accept", "silu"):
        run_small_only(args)
        return
    run_gpu(args)


if __name__ == "__main__":
    main()
