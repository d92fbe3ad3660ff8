"""The allocation-free verify-attention entry point, called straight through the C ABI.

Some hosts cannot hand the kernel a scratch workspace because they cannot allocate one: all
HBM already belongs to their KV pool, or an allocation would stall a loop that must not stall.
`rlt_verify_attention_noalloc` scores the same inputs on a fixed block of device memory that
ships inside the library.  This file checks, on calls in a row that share that block, that its
output is bit-identical to the workspace-taking entry point and within tolerance of the CPU
oracle (also on the second call, which finds the block dirty), that a warmed-up call leaves the
device's memory accounting untouched, and that a batch too large for the block is refused before
anything is launched.

Collected last on purpose (the file name sorts after every other test file), and written so
that it passes both on its own in a fresh process and after the rest of the suite.
"""

import ctypes

import pytest
import torch

from helpers import make_pool
from oracle import oracle
from vllm_rlt_b200 import _capi

pytestmark = pytest.mark.gpu


def call_entry(lib, name, q, key, value, tables, lengths, workspace=None, cu=None):
    out = torch.empty_like(q)
    blocks, block_size, kv_heads, head_dim = key.shape
    args = [_capi.ptr(q), _capi.ptr(out), _capi.ptr(key), _capi.ptr(value), key.stride(0), key.stride(1), blocks,
            block_size, q.shape[1], kv_heads, head_dim, _capi.DTYPE_CODES[q.dtype], _capi.ptr(tables),
            tables.shape[0], tables.shape[1], _capi.ptr(lengths), _capi.ptr(cu), q.shape[0]]
    if workspace is not None:
        args += [_capi.ptr(workspace), workspace.numel()]
    args.append(_capi.stream_of(q))
    status = getattr(lib, name)(*args)
    return status, out


def make_case(seed, contexts, rows_per_request, dtype=torch.bfloat16):
    row_lengths = [[c - rows_per_request + 1 + t for t in range(rows_per_request)] for c in contexts]
    pool = make_pool(contexts, kv_heads=16, head_dim=128, block=16, dtype=dtype, seed=seed, layers=2,
                     layer=1, row_lengths=row_lengths)
    g = torch.Generator().manual_seed(seed + 100)
    q = (torch.randn(pool["tables"].shape[0], 16, 128, generator=g) * 0.5).to(dtype)
    key, value = pool["key_pool"].cuda()[:, 1], pool["value_pool"].cuda()[:, 1]
    return dict(q=q.cuda(), key=key, value=value, tables=pool["tables"].cuda(), lengths=pool["lengths"].cuda(),
                host=(q, pool["key"], pool["value"], pool["tables"], pool["lengths"]))


def oracle_of(case, lengths=None):
    q, key, value, tables, host_lengths = case["host"]
    return oracle.paged_attention(q, key, value, tables.clamp_min(0), host_lengths if lengths is None else lengths).float()


def test_a_zero_row_call_is_the_warm_up_and_launches_nothing():
    # the first thing this process asks of the entry point: the set-up a host performs once per device,
    # before it gives its remaining memory away
    lib = _capi.load()
    torch.cuda.set_device(0)
    q = torch.empty(0, 16, 128, dtype=torch.bfloat16, device="cuda")
    key = torch.zeros(2, 16, 16, 128, dtype=torch.bfloat16, device="cuda")
    tables = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    lengths = torch.zeros(1, dtype=torch.int32, device="cuda")
    status, _ = call_entry(lib, "rlt_verify_attention_noalloc", q, key, key, tables, lengths)
    assert status == 0, _capi.last_error()
    torch.cuda.synchronize()


def test_noalloc_entry_matches_the_workspace_entry_on_two_calls_in_a_row():
    lib = _capi.load()
    torch.cuda.set_device(0)
    # call 1 leaves multi-chunk partials, counters and a work list behind in the shared block;
    # call 2 is a different batch (other groups, other lengths, an empty row) on the same block.
    cases = [make_case(1, [1300, 40, 700], 5), make_case(2, [90, 2100], 7)]
    cases[1]["lengths"][3] = 0  # one empty row in the second batch
    host_lengths = cases[1]["host"][4].clone()
    host_lengths[3] = 0
    for case, lengths in zip(cases, (None, host_lengths)):
        q, key, value, tables = case["q"], case["key"], case["value"], case["tables"]
        need = lib.rlt_verify_attention_workspace_bytes(q.shape[0], 16, 16, 128, 16, tables.shape[1])
        workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        status, want = call_entry(lib, "rlt_verify_attention", q, key, value, tables, case["lengths"], workspace)
        assert status == 0, _capi.last_error()
        status, got = call_entry(lib, "rlt_verify_attention_noalloc", q, key, value, tables, case["lengths"])
        assert status == 0, _capi.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert bool(torch.isfinite(got.float()).all())
        # independent of the sibling entry: the CPU oracle, on the clean and on the dirty block
        torch.testing.assert_close(got.float().cpu(), oracle_of(case, lengths), rtol=2e-2, atol=2e-2)
    assert torch.count_nonzero(got[3]) == 0


def test_back_to_back_calls_on_one_stream_allocate_nothing():
    lib = _capi.load()
    torch.cuda.set_device(0)
    first, second = make_case(3, [600, 33], 4), make_case(4, [75, 1500, 20], 6, dtype=torch.float16)
    packed = make_case(5, [900, 130], 5)
    for case in (first, second, packed):                   # warm-up: every kernel variant is loaded, scratch resolved
        call_entry(lib, "rlt_verify_attention_noalloc", case["q"], case["key"], case["value"], case["tables"], case["lengths"])
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    results = []
    for case in (first, second):                           # two different batches, no host synchronisation between them
        results.append(call_entry(lib, "rlt_verify_attention_noalloc", case["q"], case["key"], case["value"],
                                  case["tables"], case["lengths"]))
    # the packed form (one table row per request, cu_seqlens_q) through the same entry
    tables = packed["tables"][::5].contiguous()
    context = packed["lengths"][4::5].contiguous()
    cu = (torch.arange(3, device="cuda") * 5).int()
    packed_status, packed_out = call_entry(lib, "rlt_verify_attention_noalloc", packed["q"], packed["key"], packed["value"],
                                           tables, context, cu=cu)
    torch.cuda.synchronize()
    # nothing but the outputs this test itself allocated (call_entry's empty_like) came from any allocator
    output_bytes = sum(t.numel() * t.element_size() for t in (first["q"], second["q"], packed["q"]))
    assert torch.cuda.memory_allocated() - allocated_before <= output_bytes + 3 * 512
    assert free_before - torch.cuda.mem_get_info()[0] <= max(output_bytes, 2 << 20) + (2 << 20)
    for (status, got), case, tolerance in zip(results, (first, second), (2e-2, 2e-3)):
        assert status == 0, _capi.last_error()
        torch.testing.assert_close(got.float().cpu(), oracle_of(case), rtol=tolerance, atol=tolerance)
    assert packed_status == 0, _capi.last_error()
    torch.testing.assert_close(packed_out.float().cpu(), oracle_of(packed), rtol=2e-2, atol=2e-2)


def test_noalloc_entry_refuses_batches_beyond_its_block():
    lib = _capi.load()
    torch.cuda.set_device(0)
    rows, width = 1024, 256  # needs about 70 MB of scratch: more than the 32 MiB block
    q = torch.zeros(rows, 16, 128, dtype=torch.bfloat16, device="cuda")
    key = torch.zeros(8, 16, 16, 128, dtype=torch.bfloat16, device="cuda")
    tables = torch.zeros(rows, width, dtype=torch.int32, device="cuda")
    lengths = torch.ones(rows, dtype=torch.int32, device="cuda")
    assert lib.rlt_verify_attention_workspace_bytes(rows, 16, 16, 128, 16, width) > 32 << 20
    status, _ = call_entry(lib, "rlt_verify_attention_noalloc", q, key, key, tables, lengths)
    assert status == _capi.ERR_WORKSPACE
    assert "built-in scratch" in _capi.last_error()
    torch.cuda.synchronize()
