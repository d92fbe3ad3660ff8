"""Benchmark of the self-speculative verify step on B200 (and its CPU baseline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One *step* is one pass of the verify hot path over one batch of synthetic input at the
kernel-microbench shape of BASELINE.json (configs[1]) extended over the 24 layers of the
Ouro-1.4B shape:

    for each of 24 layers:  KV write of the new tokens -> grouped paged verify attention
                            (64 requests, 16 heads x 128, 16-token pages, contexts U[512, 4096],
                             16 rows per request = 4 tokens x 4 loop depths, shared depth plane)
                         -> SiLU-and-Mul on [1024, 5632]
    then                    greedy acceptance and rejection-sampling acceptance (T = 0.8) on
                            64 x 4 rows of 49152 fp32 logits, and the device rollback.

The model GEMMs / norms / RoPE between these calls are not part of the path and are not run.
`value` is accepted tokens per second (device-resident inputs); committed tokens (accepted + 1
per request) are reported beside it.  `e2e` is the same step driven from pinned host buffers
through the public Python API (H2D of every input and D2H of the result inside the timed
region).  One process per GPU; every rank runs an independent replica on its own requests
(no collective on the path), the timed region is bracketed by a barrier, and the step time is
the maximum over ranks.

Other entry points (each prints its own JSON line; none is the contract line above):
    --workload decode [--requests R --output-tokens T --temperature X --eager --prompt-min A --prompt-max B
                       --shared-prefix P --prefix-caching]
                      whole-model self-speculative decoding of a random-init Ouro-1.4B-shaped model
                      (BASELINE configs[2]) with its HBM roofline
    --only attention  [--requests --layers --tokens --depths --kv-heads --context-min --context-max --shared-plan]
    --only prefill    [--requests --tokens --kv-heads --eager]   packed causal prefill, TFLOP/s
    --only accept | --only silu                                  the small kernels at the step's shapes
"""

from __future__ import annotations

import argparse
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
METRIC = "accepted tokens/s/GPU, Ouro-1.4B self-spec decode; verify-attn % HBM peak"
# DRAM bytes (read + write) per algorithmic byte of verify_attention_kernel, from the ncu capture
# summarised in profiles/verify_attention_kernel_config2.md (32-request case; traffic grows in
# proportion to the K/V read, so the ratio carries over to a full launch).
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


def bind_to_gpu_numa_node(local: int):
    """Runs this process on the cores of the NUMA node its GPU hangs off (sysfs; a process
    setting, nothing of the GPU's changes), so that the pinned staging buffers of the host-driven
    step are first touched — and therefore placed — in that node's memory.  With several replicas
    per machine the uploads otherwise share one node's memory channels and the socket link.
    Returns the node, or None when the topology cannot be read."""
    try:
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        domain = torch.cuda.get_device_properties(local).pci_domain_id
        device_id = torch.cuda.get_device_properties(local).pci_device_id
        path = f"/sys/bus/pci/devices/{domain:04x}:{bus:02x}:{device_id:02x}.0/numa_node"
        node = int(open(path).read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError):
        return None


def run_gpu(args):
    import torch.distributed as dist

    import vllm_rlt_b200 as rlt

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    work = Workload(seed=replica_seed(rank))
    host = work.host_inputs(pin=True)
    dev = {name: t.to(device) for name, t in host.items()}
    g = torch.Generator(device=device).manual_seed(99 + rank)
    pool_shape = (work.total_pages, LAYERS, BLOCK, HEADS, HEAD_DIM)
    key_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
    value_pool = torch.empty(pool_shape, dtype=torch.bfloat16, device=device)
    for pool in (key_pool, value_pool):  # N(0,1) * 0.5, generated in slabs to bound temporaries
        flat = pool.view(-1)
        step = 1 << 28
        for start in range(0, flat.numel(), step):
            n = min(step, flat.numel() - start)
            flat[start:start + n] = (torch.randn(n, device=device, generator=g) * 0.5).to(torch.bfloat16)
    backend = rlt.create_backend(device, torch.bfloat16, HEAD_DIM, BLOCK)
    slot_values = torch.zeros(2 * work.requests, 2, dtype=torch.int64, device=device)
    per_row_t = dev["temperature"].repeat_interleave(TOKENS)
    launches = 0
    attn_events = []

    def hot_path(x, timed_attention, before_layer=None, before_accept=None):
        """One verify pass on device tensors `x`; returns (result buffer, rollback state).
        The two hooks let a host-driven caller wait for that layer's / the logits' upload."""
        nonlocal launches
        # all layers of the pass share the block tables and lengths: plan once, run per layer
        with backend.kernel.shared_plan():
            for layer in range(LAYERS):
                if before_layer is not None:
                    before_layer(layer)
                kc, vc = key_pool[:, layer], value_pool[:, layer]
                rlt.kv_write(kc, vc, x["k"][layer], x["v"][layer], x["write_blocks"], x["write_offsets"])
                if timed_attention:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                backend(x["q"][layer], kc, vc, x["tables"], x["lengths"])
                if timed_attention:
                    b.record()
                    attn_events.append((a, b))
                rlt.silu_and_mul(x["gate"][layer], x["up"][layer])
                launches += 3  # kv_write, attention, silu_and_mul
        launches += 1  # the pass's one attention plan
        if before_accept is not None:
            before_accept()
        # drafts proposed from q with the explicit-uniform rule, then both acceptance modes
        drafts, _ = rlt.sample_rows(x["draft"], per_row_t, x["u_draft"])
        tokens = torch.zeros(work.requests, TOKENS, dtype=torch.int64, device=device)
        tokens[:, 1:] = drafts.view(work.requests, TOKENS)[:, :-1]
        rlt.accept_greedy(x["target"], x["cu_rows"], tokens, x["starts"], x["slots"], slot_values)
        result, _ = rlt.accept_rejection(x["target"], x["draft"], x["cu_rows"], tokens, x["starts"],
                                         x["temperature"], x["u_accept"], x["u_final"], x["slots"], slot_values)
        accepted = result[work.accept_rows:work.accept_rows + work.requests]
        rolled = rlt.rollback(x["starts"], accepted + 1, x["request_tables"], BLOCK)
        launches += 6  # sample_rows, argmax + greedy finish, row stats + decide (rejection), rollback
        return result, rolled

    # ---- device-resident timing ----
    for _ in range(args.warmup):
        hot_path(dev, False)
    barrier()
    launches = 0
    clocks = ClockSampler(local)
    clocks.__enter__()  # samples until the end of the second (host-driven) timed region
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        result, _ = hot_path(dev, True)
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    launches_per_step = launches // args.steps
    attention_ms = statistics.mean(a.elapsed_time(b) for a, b in attn_events)
    accepted_per_step = int(result[work.accept_rows:work.accept_rows + work.requests].sum())
    committed_per_step = accepted_per_step + work.requests

    # ---- end to end from pinned host buffers through the public API ----
    # Every step uploads all of its inputs from pinned host memory and reads its result back.
    # Uploads run on a copy stream, layer by layer, into one of two staging sets, so the copy of
    # layer l+1 (and of the next step) overlaps the kernels of layer l; the compute stream waits
    # for exactly the tensors it is about to read.
    per_layer = ("q", "k", "v", "gate", "up")
    last = ("target", "draft")
    first = [name for name in host if name not in per_layer + last]
    sets = [{name: torch.empty_like(t, device=device) for name, t in host.items()} for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=device)
    compute_stream = torch.cuda.current_stream(device)
    set_free = [None, None]  # event: the compute that used this staging set has finished
    result_host = torch.empty(work.accept_rows + 2 * work.requests, dtype=torch.int64).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = result_host.numel() * 8
    e2e_counter = 0

    def e2e_step():
        nonlocal e2e_counter
        which = e2e_counter % 2
        e2e_counter += 1
        staged = sets[which]
        layer_ready = [torch.cuda.Event() for _ in range(LAYERS)]
        first_ready, last_ready = torch.cuda.Event(), torch.cuda.Event()
        with torch.cuda.stream(copy_stream):
            if set_free[which] is not None:
                copy_stream.wait_event(set_free[which])
            for name in first:
                staged[name].copy_(host[name], non_blocking=True)
            first_ready.record(copy_stream)
            for layer in range(LAYERS):
                for name in per_layer:
                    staged[name][layer].copy_(host[name][layer], non_blocking=True)
                layer_ready[layer].record(copy_stream)
            for name in last:
                staged[name].copy_(host[name], non_blocking=True)
            last_ready.record(copy_stream)
        compute_stream.wait_event(first_ready)
        result, _ = hot_path(staged, False, before_layer=lambda layer: compute_stream.wait_event(layer_ready[layer]),
                             before_accept=lambda: compute_stream.wait_event(last_ready))
        result_host.copy_(result, non_blocking=True)
        done = torch.cuda.Event()
        done.record(compute_stream)
        set_free[which] = done

    for _ in range(min(args.warmup, 3)):
        e2e_step()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e_stop.record()
    barrier()
    clocks.__exit__(None, None, None)
    e2e_ms = e_start.elapsed_time(e_stop)
    status = backend.kernel.last_status(device)

    times = torch.tensor([elapsed_ms, e2e_ms, float(accepted_per_step), float(committed_per_step)],
                         dtype=torch.float64, device=device)
    job = combine_ranks(times if world > 1 else times.cpu(), world, args.steps, all_gather_rows)
    if rank == 0:
        ms_per_step, value = job["ms_per_step"], job["accepted_tokens_per_s"]
        accepted_total, committed_total = job["accepted_per_step"], job["committed_per_step"]
        peak, peak_kind = measured_peaks()
        algorithmic = work.algorithmic_attention_bytes()
        achieved = algorithmic / (attention_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "accepted tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": "configs[1] verify-step microbench x 24 layers: 64 requests/GPU, 16x128 MHA, "
                            "block 16, ctx U[512,4096], 4 tokens x 4 depths shared plane, bf16; sampler 256 rows x "
                            "49152 fp32 (greedy + rejection T=0.8, draft = target + N(0,0.5)); rollback",
                "requests_per_gpu": work.requests, "layers": LAYERS, "attention_rows": work.rows,
                "kv_pool_gb": round(2 * key_pool.numel() * 2 / 1e9, 2),
                "l2_policy": "inputs larger than L2 (KV pool streamed once per step)",
                "parallelism": f"{world} independent replicas, no collective",
                "host_numa_node_rank0": numa,
            },
            "committed_tokens_per_s": job["committed_tokens_per_s"],
            "acceptance_rate": accepted_total / (world * work.requests * (TOKENS - 1)),
            "e2e": {"value": job["e2e_accepted_tokens_per_s"], "unit": "accepted tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": job["e2e_ms_per_step"]},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "kernel": "verify_attention_kernel (per layer call; one plan per 24-layer pass amortised in)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ATTENTION_TRAFFIC_RATIO * algorithmic,
                         "traffic_source": "ncu dram bytes of a 32-request launch scaled by algorithmic bytes",
                         "algorithmic_bytes": algorithmic,
                         "avg_launch_ms": attention_ms},
            "clocks": clocks.summary(),
            "attention_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(threads=os.cpu_count() or 1, budget_s=12.0)
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
        g = torch.Generator(device=device).manual_seed(3)
        gate = (torch.randn(work.rows, FFN, device=device, generator=g) * 3).to(torch.bfloat16)
        up = torch.randn(work.rows, FFN, device=device, generator=g).to(torch.bfloat16)
        ms = timed(lambda: rlt.silu_and_mul(gate, up))
        nbytes = 3 * gate.numel() * 2
        out.update(rows=work.rows, ms=ms, bytes=nbytes, gbs=nbytes / ms / 1e6)
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
    through `vllm_rlt_b200.SelfSpeculativeDecoder` — BASELINE configs[2] with the output length set by
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
    if args.shared_prefix > 0:   # every second request starts with one common prefix (BASELINE configs[4]'s mix)
        common = torch.randint(1, config.vocab_size, (args.shared_prefix,), generator=g).tolist()
        prompts = [common[:len(p) - 1] + p[len(common[:len(p) - 1]):] if i % 2 else p for i, p in enumerate(prompts)]
    decoder = rlt.SelfSpeculativeDecoder(model, cuda_graphs=not args.eager, prefix_caching=args.prefix_caching)
    clock = {}

    def start_clock():
        torch.cuda.synchronize()
        clock["start"] = time.perf_counter()

    torch.cuda.synchronize()
    clock["begin"] = time.perf_counter()
    tokens = decoder.generate(prompts, args.output_tokens, num_speculative_tokens=4, draft_loops=2, target_loops=4,
                              temperature=args.temperature, seed=1, after_prefill=start_clock)
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
    head_calls = stats.rounds / max(args.requests, 1) * 5          # upper bound: k draft calls + 1 verify call per round
    head_bytes = 2.0 * c.vocab_size * c.hidden_size * head_calls
    peak, peak_kind = measured_peaks()
    roofline_s = (weight_bytes + kv_bytes + head_bytes) / (peak * 1e9)
    print(json.dumps({
        "workload": "decode: Ouro-1.4B-shaped random-init bf16, self-spec k=4 from depth 2, "
                    f"{args.requests} requests, prompts U[{args.prompt_min},{args.prompt_max}]"
                    + (f" (every second one behind a common {args.shared_prefix}-token prefix, prefix reuse "
                       f"{'on' if args.prefix_caching else 'off'})" if args.shared_prefix else "")
                    + f", {args.output_tokens} output tokens, T={args.temperature}, "
                    + ("eager launches" if args.eager else "recurrent loops replayed from CUDA graphs"),
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


def cpu_step_seconds(threads: int, budget_s: float):
    """Times the CPU oracle on a bounded sample of the same workload and extrapolates linearly
    to one full step.  Returns (estimated seconds per step, accepted tokens per step, sample text)."""
    from oracle import oracle

    torch.set_num_threads(threads)
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    sample_requests = 32
    work = Workload(seed=1234, requests=sample_requests, layers=1)
    x = work.host_inputs(pin=False)
    g = torch.Generator().manual_seed(5)
    pool_shape = (work.total_pages, 1, BLOCK, HEADS, HEAD_DIM)
    key_pool = (torch.randn(pool_shape, generator=g) * 0.5).bfloat16()
    value_pool = (torch.randn(pool_shape, generator=g) * 0.5).bfloat16()
    kc, vc = key_pool[:, 0], value_pool[:, 0]

    def one_layer():
        t = time.perf_counter()
        oracle.kv_write(kc, vc, x["k"][0], x["v"][0], x["write_blocks"], x["write_offsets"])
        oracle.paged_attention(x["q"][0], kc, vc, x["tables"], x["lengths"])
        oracle.silu_and_mul(x["gate"][0], x["up"][0])
        return time.perf_counter() - t

    # The layers differ only in their data: time as many passes of one layer as fit the budget.
    times = [one_layer()]
    sample_layers = max(1, min(LAYERS, int(budget_s / max(times[0], 1e-3))))
    times += [one_layer() for _ in range(sample_layers - 1)]
    layer_s = statistics.mean(times)
    t1 = time.perf_counter()
    per_row_t = x["temperature"].repeat_interleave(TOKENS)
    drafts, _ = oracle.sample_rows(x["draft"], per_row_t, x["u_draft"])
    tokens = torch.zeros(sample_requests, TOKENS, dtype=torch.int64)
    tokens[:, 1:] = drafts.view(sample_requests, TOKENS)[:, :-1]
    oracle.accept_greedy(x["target"], x["cu_rows"], tokens, x["starts"])
    result, _ = oracle.accept_rejection(x["target"], x["draft"], x["cu_rows"], tokens, x["starts"],
                                        x["temperature"], x["u_accept"], x["u_final"])
    accepted = result[work.accept_rows:work.accept_rows + sample_requests]
    oracle.rollback(x["starts"], accepted + 1, x["request_tables"], BLOCK)
    accept_s = time.perf_counter() - t1
    scale = REQUESTS / sample_requests
    step_s = scale * (LAYERS * layer_s + accept_s)
    acceptance = float(accepted.sum()) / (sample_requests * (TOKENS - 1))
    sample = (f"{sample_requests} of {REQUESTS} requests, {sample_layers} of {LAYERS} layers "
              f"(kv_write + attention + silu) + acceptance on {work.accept_rows} rows; "
              f"{sum(times) + accept_s:.1f} s measured, scaled x{scale:.0f} requests, layers x{LAYERS}")
    return step_s, acceptance * REQUESTS * (TOKENS - 1), sample, oracle.num_threads()


def cpu_baseline(threads: int, budget_s: float):
    step_s, accepted, sample, used = cpu_step_seconds(threads, budget_s)
    return {"value": accepted / step_s, "unit": "accepted tokens/s", "cores": used, "kind": "port",
            "sample": sample, "estimated_s_per_step": step_s}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's Torch path for this step (the
    reference package itself is Python over PyTorch and is not present on the GPU box), timed on
    all host cores; each step is the same bounded sample, scaled to a full step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        cpu_step_seconds(threads, 8.0)
    steps = max(1, min(args.steps, 3))
    results = [cpu_step_seconds(threads, 8.0) for _ in range(steps)]
    step_s = statistics.mean(r[0] for r in results)
    accepted, sample, used = results[0][1], results[0][2], results[0][3]
    value = accepted / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "accepted tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[1] verify-step microbench x 24 layers (CPU, bounded sample scaled to a full step)"},
        "cpu_baseline": {"value": value, "unit": "accepted tokens/s", "cores": used, "kind": "port", "sample": sample},
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
    parser.add_argument("--workload", default="step", choices=["step", "decode"],
                        help="step: the verify-step microbench (the bench line); decode: whole-model decoding (secondary)")
    parser.add_argument("--output-tokens", type=int, default=32)
    parser.add_argument("--eager", action="store_true", help="decode workload: launch every kernel from the host")
    parser.add_argument("--prompt-min", type=int, default=128, help="decode workload: shortest prompt")
    parser.add_argument("--prompt-max", type=int, default=1024, help="decode workload: longest prompt")
    parser.add_argument("--shared-prefix", type=int, default=0,
                        help="decode workload: every second prompt starts with one common prefix of this many tokens")
    parser.add_argument("--prefix-caching", action="store_true", help="decode workload: map shared prompt pages instead of recomputing them")
    parser.add_argument("--temperature", type=float, default=0.8)
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
    if args.workload == "decode":
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
