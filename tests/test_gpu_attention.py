"""Verify attention on the GPU vs the CPU oracle, the golden vectors of the reference, and
its own invariance contract (a row's bits do not depend on its batch or its group).

Tolerances: bf16 2e-2 and fp16 2e-3 (the reference's own GPU tolerances,
tests/test_attention.py:54 there), fp32 1e-5 relative.
"""

import pytest
import torch

import vllm_rlt_b200 as rlt
from helpers import attention_tolerance, make_pool
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kernel():
    return rlt.B200PagedAttention()


def run_gpu(kernel, q, key_pool, value_pool, layer, tables, lengths, cu=None):
    k = key_pool.cuda()[:, layer]
    v = value_pool.cuda()[:, layer]
    if cu is None:
        out = kernel(q.cuda(), k, v, tables.cuda(), lengths.cuda())
    else:
        out = kernel.prefill(q.cuda(), k, v, tables.cuda(), lengths.cuda(), cu.cuda(), 0)
    torch.cuda.synchronize()
    return out.cpu()


def chunk_count(length):
    """Python mirror of the kernel's fixed context chunking (512-token chunks up to 8192,
    then four chunks per power-of-two octave)."""
    if length <= 0:
        return 0
    if length <= 8192:
        return -(-length // 512)
    k = ((length - 1) >> 13).bit_length() - 1
    return 16 + 4 * k + (length - 1 - (8192 << k)) // (2048 << k) + 1


def check(got, want, dtype):
    tol = attention_tolerance(dtype)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=tol, atol=tol)
    else:
        torch.testing.assert_close(got.float(), want.float(), rtol=tol, atol=tol)


def test_golden_vectors_of_the_reference(kernel, golden):
    for case in golden("attention.pt"):
        if case["kind"] == "direct":
            k, v = case["k"], case["v"]
        else:
            k, v = case["key_cache"][:, case["layer"]], case["value_cache"][:, case["layer"]]
        got = kernel(case["q"].cuda(), k.cuda(), v.cuda(), case["tables"].cuda(), case["lengths"].cuda()).cpu()
        check(got, case["out"], case["q"].dtype)
        for row in (case["lengths"] == 0).nonzero().flatten().tolist():
            assert torch.count_nonzero(got[row]) == 0


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,block", [
    (torch.float32, 4, 4, 64, 16),     # the tiny fp32 model of config 1
    (torch.float32, 6, 2, 7, 2),
    (torch.float16, 8, 8, 96, 16),
    (torch.bfloat16, 6, 2, 32, 4),
])
def test_generic_shapes_match_oracle(kernel, dtype, heads, kv_heads, dim, block):
    pool = make_pool([71, 5, 33, 64, 1], kv_heads=kv_heads, head_dim=dim, block=block, dtype=dtype, seed=11,
                     layers=2, layer=1, row_lengths=[[1, 32, 71], [5], [33, 17], [64], [1]], scale=1.0)
    g = torch.Generator().manual_seed(12)
    q = torch.randn(pool["tables"].shape[0], heads, dim, generator=g).to(dtype)
    got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 1, pool["tables"], pool["lengths"])
    want = oracle.paged_attention(q, pool["key"], pool["value"], pool["tables"].clamp_min(0), pool["lengths"])
    check(got, want, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", ["shared", "last_exited", "verify"])
def test_tiled_kernel_matches_oracle_on_verify_shapes(kernel, dtype, layout):
    # Scaled-down config 2: requests with 16 heads x 128, 16-token pages, permuted pool, layer-strided view.
    g = torch.Generator().manual_seed(77)
    contexts = torch.randint(40, 1500, (6,), generator=g).tolist() + [512, 513]
    if layout == "shared":       # 4 tokens x 4 depths share one table; row (t, depth) sees ctx - 3 + t
        groups = contexts
        row_lengths = [[c - 3 + t for _ in range(4) for t in range(4)] for c in contexts]
    elif layout == "last_exited":  # one table per (request, depth plane), 4 rows each
        groups = [c for c in contexts for _ in range(4)]
        row_lengths = [[c - 3 + t for t in range(4)] for c in contexts for _ in range(4)]
    else:                        # the real verify shape: k + 1 = 5..7 rows per request
        groups = contexts
        row_lengths = [[c - n + 1 + t for t in range(n)] for c, n in zip(contexts, [5, 6, 7, 5, 6, 7, 5, 5])]
    pool = make_pool(groups, kv_heads=16, head_dim=128, block=16, dtype=dtype, seed=5, layers=3, layer=2,
                     row_lengths=row_lengths)
    q = (torch.randn(pool["tables"].shape[0], 16, 128, generator=g) * 0.5).to(dtype)
    got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 2, pool["tables"], pool["lengths"])
    want = oracle.paged_attention(q, pool["key"], pool["value"], pool["tables"].clamp_min(0), pool["lengths"])
    check(got, want, dtype)
    # Every group was found (its K/V is streamed once, not once per row) and no wait gave up.
    status = kernel.last_status()
    assert status["error"] == 0 and status["claim_counter"] == 0
    assert status["items"] == sum(16 * chunk_count(max(lengths)) for lengths in row_lengths)


def test_long_contexts_use_octave_chunks(kernel):
    dtype = torch.bfloat16
    row_lengths = [[8190, 8191, 8192, 8193, 8194], [20000], [40003, 40004]]
    pool = make_pool([8194, 20000, 40004], kv_heads=2, head_dim=128, block=16, dtype=dtype, seed=13,
                     row_lengths=row_lengths)
    g = torch.Generator().manual_seed(14)
    q = torch.randn(pool["tables"].shape[0], 4, 128, generator=g).to(dtype)
    got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, pool["tables"], pool["lengths"])
    want = oracle.paged_attention(q, pool["key"], pool["value"], pool["tables"].clamp_min(0), pool["lengths"])
    check(got, want, dtype)
    status = kernel.last_status()
    assert status["error"] == 0
    assert status["items"] == 2 * (chunk_count(8194) + chunk_count(20000) + chunk_count(40004))
    for row in (0, 3, 5, 7):
        one = slice(row, row + 1)
        alone = run_gpu(kernel, q[one], pool["key_pool"], pool["value_pool"], 0, pool["tables"][one],
                        pool["lengths"][one])
        assert torch.equal(alone[0], got[row]), row


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_split_kv_boundaries_and_batch_invariance(kernel, dtype):
    # Empty row, page, chunk and octave boundaries, GQA 2 (tests/test_attention.py:154-184 of the reference).
    lengths = [0, 1, 15, 16, 17, 511, 512, 513, 1024, 4096, 4097, 5121, 10000]
    pool = make_pool(lengths, kv_heads=4, head_dim=128, block=16, dtype=dtype, seed=1, scale=1.0, pad=0)
    g = torch.Generator().manual_seed(2)
    q = torch.randn(len(lengths), 8, 128, generator=g).to(dtype)
    got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, pool["tables"], pool["lengths"])
    want = oracle.paged_attention(q, pool["key"], pool["value"], pool["tables"], pool["lengths"])
    check(got, want, dtype)
    assert torch.count_nonzero(got[0]) == 0
    for row in (1, 5, 8, 10, 12):
        one = slice(row, row + 1)
        alone = run_gpu(kernel, q[one], pool["key_pool"], pool["value_pool"], 0, pool["tables"][one],
                        pool["lengths"][one])
        assert torch.equal(alone[0], got[row]), row


def test_row_bits_do_not_depend_on_group_membership(kernel):
    # The k+1 rows of a request scored as one group, one by one, and through the packed
    # interface must agree bit for bit; lengths straddle a chunk boundary on purpose.
    dtype = torch.bfloat16
    contexts = [515, 1030, 64, 4100]
    rows_per = [7, 5, 6, 4]
    row_lengths = [[c - n + 1 + t for t in range(n)] for c, n in zip(contexts, rows_per)]
    pool = make_pool(contexts, kv_heads=16, head_dim=128, block=16, dtype=dtype, seed=3, row_lengths=row_lengths)
    g = torch.Generator().manual_seed(4)
    rows = sum(rows_per)
    q = (torch.randn(rows, 16, 128, generator=g) * 0.5).to(dtype)
    grouped = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, pool["tables"], pool["lengths"])
    for row in range(rows):
        one = slice(row, row + 1)
        alone = run_gpu(kernel, q[one], pool["key_pool"], pool["value_pool"], 0, pool["tables"][one],
                        pool["lengths"][one])
        assert torch.equal(alone[0], grouped[row]), row
    # packed: one table row per request, cu_seqlens_q, length of the last row
    first_rows = [sum(rows_per[:i]) for i in range(len(rows_per))]
    seq_tables = pool["tables"][first_rows]
    seq_lengths = torch.tensor(contexts, dtype=torch.int32)
    cu = torch.tensor(first_rows + [rows], dtype=torch.int32)
    packed = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, seq_tables, seq_lengths, cu)
    assert torch.equal(packed, grouped)
    # a shuffled batch of the same rows (groups broken up) still gives the same bits
    perm = torch.randperm(rows, generator=g)
    shuffled = run_gpu(kernel, q[perm], pool["key_pool"], pool["value_pool"], 0, pool["tables"][perm],
                       pool["lengths"][perm])
    assert torch.equal(shuffled, grouped[perm])


def test_shared_plan_runs_every_layer_with_one_plan(kernel):
    # One plan, many runs: every layer of a pass shares block tables and lengths.  The result of
    # each layer must equal the self-planned call bit for bit, including zero-length rows and
    # multi-chunk rows (whose counters and claim counter must be left clean by every run).
    dtype = torch.bfloat16
    row_lengths = [[1290, 1291, 1292], [0], [33, 34], [513]]
    pool = make_pool([1292, 16, 34, 513], kv_heads=16, head_dim=128, block=16, dtype=dtype, seed=21, layers=3,
                     row_lengths=row_lengths)
    g = torch.Generator().manual_seed(22)
    rows = pool["tables"].shape[0]
    qs = [(torch.randn(rows, 16, 128, generator=g) * 0.5).to(dtype).cuda() for _ in range(3)]
    kp, vp = pool["key_pool"].cuda(), pool["value_pool"].cuda()
    tables, lengths = pool["tables"].cuda(), pool["lengths"].cuda()
    separate = [kernel(qs[layer], kp[:, layer], vp[:, layer], tables, lengths) for layer in range(3)]
    with kernel.shared_plan():
        shared = [kernel(qs[layer], kp[:, layer], vp[:, layer], tables, lengths) for layer in range(3)]
        again = kernel(qs[0], kp[:, 0], vp[:, 0], tables, lengths)
        status = kernel.last_status()
    torch.cuda.synchronize()
    for layer in range(3):
        assert torch.equal(shared[layer], separate[layer]), layer
    assert torch.equal(again, separate[0])
    assert status["error"] == 0 and status["zero_rows"] == 1 and status["claim_counter"] == 0
    assert torch.count_nonzero(shared[1][3]) == 0
    # different lengths tensor inside the context -> replanned, not reused
    shorter = (lengths - 1).clamp_min(0)
    with kernel.shared_plan():
        a = kernel(qs[0], kp[:, 0], vp[:, 0], tables, lengths)
        b = kernel(qs[0], kp[:, 0], vp[:, 0], tables, shorter)
    assert torch.equal(a, separate[0])
    assert torch.equal(b, kernel(qs[0], kp[:, 0], vp[:, 0], tables, shorter))


def test_padding_entries_are_never_dereferenced(kernel):
    dtype = torch.bfloat16
    pool = make_pool([40, 300, 17], kv_heads=2, head_dim=128, block=16, dtype=dtype, seed=6,
                     row_lengths=[[38, 39, 40], [300], [0, 17]])
    g = torch.Generator().manual_seed(7)
    q = torch.randn(pool["tables"].shape[0], 4, 128, generator=g).to(dtype)
    clean = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, pool["tables"].clamp_min(0), pool["lengths"])
    for filler in (-1, 2**31 - 1):
        tables = pool["tables"].clone()
        tables[tables < 0] = filler
        tables[4] = filler  # the zero-length row's whole table is garbage
        got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, tables, pool["lengths"])
        assert torch.equal(got, clean)
    assert torch.count_nonzero(clean[4]) == 0


def test_empty_batch_and_argument_errors(kernel):
    k = torch.zeros(4, 16, 2, 128, device="cuda", dtype=torch.bfloat16)
    empty = kernel(torch.empty(0, 4, 128, device="cuda", dtype=torch.bfloat16), k, k,
                   torch.zeros(0, 3, dtype=torch.int32, device="cuda"), torch.zeros(0, dtype=torch.int32, device="cuda"))
    assert empty.shape == (0, 4, 128)
    q = torch.ones(1, 3, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="positive multiple"):
        kernel(q, k, k, torch.zeros(1, 1, dtype=torch.int32, device="cuda"), torch.ones(1, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError, match="int32"):
        kernel(q[:, :2], k, k, torch.zeros(1, 1, dtype=torch.int64, device="cuda"),
               torch.ones(1, dtype=torch.int32, device="cuda"))


def test_backend_adapter_and_capabilities():
    backend = rlt.create_backend("cuda", torch.bfloat16, 128, 16)
    assert backend.info["selected_backend"] == "b200" and backend.info["tiled_kernel"]
    caps = backend.capabilities
    assert caps.cuda_graphs and caps.async_scheduling and caps.device_context_lengths
    assert caps.packed_prefill and caps.packed_matches_decode and caps.sliding_window
    with pytest.raises(NotImplementedError, match="sliding-window"):       # an adapter around a kernel without the entry
        rlt.attention.AttentionBackend(lambda *a: None, caps, {"selected_backend": "plain"}).windowed()
    with pytest.raises(ValueError, match="CUDA"):
        rlt.create_backend("cpu", torch.bfloat16, 128, 16)


def test_int32_block_ids_use_64bit_physical_offsets(kernel):
    # tests/test_attention_64bit.py of the reference: offset 2**31 elements.
    if torch.cuda.mem_get_info()[0] < 9 * 2**30:
        pytest.skip("needs 9 GiB of free device memory")
    shape, strides = (2049, 1, 1, 16), (2**20, 16, 16, 1)
    key = torch.empty_strided(shape, strides, device="cuda", dtype=torch.float16)
    value = torch.empty_strided(shape, strides, device="cuda", dtype=torch.float16)
    key[0].zero_()
    value[0].fill_(-3)
    key[2048].fill_(1)
    expected = torch.arange(16, device="cuda", dtype=torch.float16).view(1, 1, 16)
    value[2048].copy_(expected)
    query = torch.ones((1, 1, 16), device="cuda", dtype=torch.float16)
    table = torch.tensor([[2048]], device="cuda", dtype=torch.int32)
    lengths = torch.tensor([1], device="cuda", dtype=torch.int32)
    torch.testing.assert_close(kernel(query, key, value, table, lengths), expected, rtol=0, atol=0)


def test_graph_capture_and_replay_with_device_lengths(kernel):
    dtype = torch.bfloat16
    pool = make_pool([600, 90], kv_heads=16, head_dim=128, block=16, dtype=dtype, seed=9,
                     row_lengths=[[596, 597, 598, 599, 600], [86, 87, 88, 89, 90]])
    g = torch.Generator().manual_seed(10)
    q = (torch.randn(10, 16, 128, generator=g) * 0.5).to(dtype).cuda()
    k, v = pool["key_pool"].cuda()[:, 0], pool["value_pool"].cuda()[:, 0]
    tables, lengths = pool["tables"].cuda(), pool["lengths"].cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            kernel(q, k, v, tables, lengths)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = kernel(q, k, v, tables, lengths)
    # new device-side lengths are picked up by a replay without any host involvement
    lengths.sub_(20)
    graph.replay()
    torch.cuda.synchronize()
    want = oracle.paged_attention(q.cpu(), pool["key"], pool["value"], pool["tables"].clamp_min(0), lengths.cpu())
    check(out.cpu(), want, dtype)


@pytest.mark.parametrize("seed", range(16))
def test_random_batches_match_oracle_and_replay_identically(kernel, seed):
    """Seeded random batches: group sizes 1..16 / gqa, GQA ratios 1..16, contexts from one token to
    beyond the first chunk octave, empty rows in between, fp16 or bf16, a layer-strided view, K below
    or above V in memory.  Checked against the oracle; a second run over the same plan gives the same
    bits (the plan survives a run) and so does every row scored alone."""
    g = torch.Generator().manual_seed(1000 + seed)
    dtype = (torch.bfloat16, torch.float16)[seed % 2]
    kv_heads = (1, 2, 4, 16)[int(torch.randint(0, 4, (1,), generator=g))]
    gqa = (1, 2, 4, 8, 16)[int(torch.randint(0, 5, (1,), generator=g))]
    q_heads = kv_heads * gqa
    cap = 16 // gqa
    groups = int(torch.randint(2, 9, (1,), generator=g))
    contexts, row_lengths = [], []
    for _ in range(groups):
        scale = (40, 600, 3000, 9500)[int(torch.randint(0, 4, (1,), generator=g))]
        ctx = int(torch.randint(1, scale + 1, (1,), generator=g))
        rows = int(torch.randint(1, min(cap, ctx) + 1, (1,), generator=g)) if cap > 1 else 1
        contexts.append(ctx)
        row_lengths.append([ctx - rows + 1 + t for t in range(rows)])
    layers, layer = 2, seed % 2
    pool = make_pool(contexts, kv_heads=kv_heads, head_dim=128, block=16, dtype=dtype, seed=seed, layers=layers,
                     layer=layer, row_lengths=row_lengths, pad=0 if seed % 3 else -1)
    tables, lengths = pool["tables"], pool["lengths"].clone()
    if seed % 4 == 0:                                  # an empty row inside a group breaks it in two
        lengths[int(torch.randint(0, lengths.numel(), (1,), generator=g))] = 0
    q = (torch.randn(tables.shape[0], q_heads, 128, generator=g) * 0.7).to(dtype)
    both = torch.stack([pool["key_pool"], pool["value_pool"]] if seed % 2 else [pool["value_pool"], pool["key_pool"]]).cuda()
    key, value = (both[0], both[1]) if seed % 2 else (both[1], both[0])
    args = (q.cuda(), key[:, layer], value[:, layer], tables.cuda(), lengths.cuda())
    with kernel.shared_plan():
        first = kernel(*args)
        again = kernel(*args)
    want = oracle.paged_attention(q, pool["key"], pool["value"], tables.clamp_min(0), lengths)
    check(first.cpu(), want, dtype)
    assert torch.equal(first, again)
    assert kernel.last_status()["error"] == 0
    for row in range(0, tables.shape[0], 3):
        one = slice(row, row + 1)
        alone = kernel(args[0][one], args[1], args[2], args[3][one], args[4][one])
        assert torch.equal(alone[0], first[row]), row


@pytest.mark.parametrize("dtype,dim", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_a_length_beyond_the_table_is_clamped_and_reported(kernel, dtype, dim):
    # device-side lengths are never seen by the host: a length the row's table cannot address must not
    # index past the table (tiled and generic kernels), and the tiled kernel reports it
    pool = make_pool([64, 300, 48], kv_heads=2, head_dim=dim, block=16, dtype=dtype, seed=12,
                     row_lengths=[[62, 63, 64], [300], [48]])
    width = pool["tables"].shape[1]
    capacity = width * 16
    tables = pool["tables"].clone()
    tables[tables < 0] = tables[0, 0]                 # a full-width table for every row (any valid page)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(tables.shape[0], 4, dim, generator=g).to(dtype)
    lengths = pool["lengths"].clone()
    over = lengths.clone()
    over[1], over[4] = capacity + 1, 2 ** 31 - 1
    clamped = lengths.clone()
    clamped[1] = clamped[4] = capacity
    got = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, tables, over)
    want = run_gpu(kernel, q, pool["key_pool"], pool["value_pool"], 0, tables, clamped)
    assert torch.equal(got, want)
    check(got, oracle.paged_attention(q, pool["key"], pool["value"], tables, clamped), dtype)
    if dtype == torch.bfloat16:
        kernel(q.cuda(), pool["key_pool"].cuda()[:, 0], pool["value_pool"].cuda()[:, 0], tables.cuda(), over.cuda())
        assert kernel.last_status()["error"] == 2     # bit 1: a length was clamped; bit 0 (a wait gave up) is clear
        kernel(q.cuda(), pool["key_pool"].cuda()[:, 0], pool["value_pool"].cuda()[:, 0], tables.cuda(), clamped.cuda())
        assert kernel.last_status()["error"] == 0


def test_shared_plan_notices_metadata_rewritten_in_place(kernel):
    # inside shared_plan() a plan is reused only while the metadata tensors are unmodified
    dtype = torch.bfloat16
    pool = make_pool([700, 90], kv_heads=2, head_dim=128, block=16, dtype=dtype, seed=4, rows_per_group=3)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(pool["tables"].shape[0], 4, 128, generator=g).to(dtype).cuda()
    kp, vp = pool["key_pool"].cuda(), pool["value_pool"].cuda()
    tables, lengths = pool["tables"].clamp_min(0).cuda(), pool["lengths"].cuda()
    shorter = (pool["lengths"] - 40).cuda()
    want_long = kernel(q, kp[:, 0], vp[:, 0], tables, lengths)
    want_short = kernel(q, kp[:, 0], vp[:, 0], tables, shorter)
    assert not torch.equal(want_long, want_short)
    with kernel.shared_plan():
        assert torch.equal(kernel(q, kp[:, 0], vp[:, 0], tables, lengths), want_long)
        lengths.copy_(shorter)                        # same storage, new contents
        assert torch.equal(kernel(q, kp[:, 0], vp[:, 0], tables, lengths), want_short)


def test_full_size_microbench_shape_matches_the_oracle_over_a_layer_strided_pool(kernel):
    # 64 requests, contexts U[512, 4096], 16 rows per request on a shared plane, layer 5 of a 24-layer pool
    # (34 GB): the oracle scores the rows of four requests from a host copy of their pages
    import bench

    work = bench.Workload(seed=1234)
    device = torch.device("cuda")
    g = torch.Generator(device=device).manual_seed(7)
    shape = (work.total_pages, bench.LAYERS, bench.BLOCK, bench.HEADS, bench.HEAD_DIM)
    key_pool = torch.empty(shape, dtype=torch.bfloat16, device=device)
    value_pool = torch.empty(shape, dtype=torch.bfloat16, device=device)
    layer = 5
    for pool in (key_pool, value_pool):               # only the layer under test needs values
        pool[:, layer] = (torch.randn(shape[0], *shape[2:], device=device, generator=g) * 0.5).to(torch.bfloat16)
    q = (torch.randn(work.rows, bench.HEADS, bench.HEAD_DIM, device=device, generator=g) * 0.5).to(torch.bfloat16)
    out = kernel(q, key_pool[:, layer], value_pool[:, layer], work.tables.to(device), work.lengths.to(device))
    status = kernel.last_status()
    assert status["error"] == 0 and status["zero_rows"] == 0
    chunks = sum(chunk_count(int(c)) for c in work.contexts)
    assert status["items"] == chunks * bench.HEADS                   # one group per request: K/V read once per request
    moved = [key_pool[:, layer:layer + 1], value_pool[:, layer:layer + 1]]
    parity = bench.attention_parity(work, out, q, moved[0], moved[1], requests=4)
    assert parity["ok"] and parity["rows"] == 64, parity
    del key_pool, value_pool
    torch.cuda.empty_cache()


def test_outgrown_scratch_stays_alive_for_graphs_that_captured_it(kernel):
    # a caller's CUDA graph has the kernels baked in with the scratch buffer of its capture; when a later, larger call
    # outgrows that buffer the old one must not go back to the allocator (someone else would get it while the graph
    # goes on replaying over it): replay after growth + fresh allocations still gives the captured result
    pool = make_pool([700, 300, 1200, 64], kv_heads=16, head_dim=128, block=16, dtype=torch.bfloat16, seed=41)
    g = torch.Generator().manual_seed(42)
    q = (torch.randn(4, 16, 128, generator=g) * 0.5).bfloat16().cuda()
    key, value = pool["key_pool"].cuda()[:, 0], pool["value_pool"].cuda()[:, 0]
    tables, lengths = pool["tables"].cuda(), pool["lengths"].cuda()
    fresh = rlt.B200PagedAttention()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        want = fresh(q, key, value, tables, lengths).clone()          # eager warm-up on the capture stream: scratch allocated here
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = fresh(q, key, value, tables, lengths)
        before = fresh._workspaces[(torch.cuda.current_device(), stream.cuda_stream)]
        many = (torch.randn(4096, 16, 128, generator=g) * 0.5).bfloat16().cuda()     # outgrows the scratch on the same stream
        fresh(many, key, value, tables[:1].expand(4096, -1).contiguous(), lengths[:1].expand(4096).contiguous())
        after = fresh._workspaces[(torch.cuda.current_device(), stream.cuda_stream)]
        assert after.numel() > before.numel() and any(b is before for b in fresh._retired)
        junk = [torch.full((before.numel() // 4,), float("nan"), device="cuda") for _ in range(8)]   # would land in freed scratch
        captured.zero_()
        graph.replay()
    stream.synchronize()
    assert torch.equal(captured, want) and len(junk) == 8
