"""The allocation-free verify-attention entry point, called straight through the C ABI.

Some hosts cannot hand the kernel a scratch workspace because they cannot allocate one: all
HBM already belongs to their KV pool, or an allocation would stall a loop that must not stall.
`rlt_verify_attention_noalloc` scores the same inputs on a fixed block of device memory that
ships inside the library.  This file checks, on two calls in a row that share that block,
that its output is bit-identical to the workspace-taking entry point, and that a batch too
large for the block is refused before anything is launched.

Collected last on purpose (the file name sorts after every other test file), and written so
that it passes both on its own in a fresh process and after the rest of the suite.
"""

import ctypes

import pytest
import torch

from helpers import make_pool
from vllm_rlt_b200 import _capi

pytestmark = pytest.mark.gpu


def call_entry(lib, name, q, key, value, tables, lengths, workspace=None):
    out = torch.empty_like(q)
    blocks, block_size, kv_heads, head_dim = key.shape
    args = [_capi.ptr(q), _capi.ptr(out), _capi.ptr(key), _capi.ptr(value), key.stride(0), key.stride(1), blocks,
            block_size, q.shape[1], kv_heads, head_dim, _capi.DTYPE_CODES[q.dtype], _capi.ptr(tables),
            tables.shape[0], tables.shape[1], _capi.ptr(lengths), ctypes.c_void_p(0), q.shape[0]]
    if workspace is not None:
        args += [_capi.ptr(workspace), workspace.numel()]
    args.append(_capi.stream_of(q))
    status = getattr(lib, name)(*args)
    return status, out


def make_case(seed, contexts, rows_per_request):
    row_lengths = [[c - rows_per_request + 1 + t for t in range(rows_per_request)] for c in contexts]
    pool = make_pool(contexts, kv_heads=16, head_dim=128, block=16, dtype=torch.bfloat16, seed=seed, layers=2,
                     layer=1, row_lengths=row_lengths)
    g = torch.Generator().manual_seed(seed + 100)
    q = (torch.randn(pool["tables"].shape[0], 16, 128, generator=g) * 0.5).to(torch.bfloat16)
    key, value = pool["key_pool"].cuda()[:, 1], pool["value_pool"].cuda()[:, 1]
    return q.cuda(), key, value, pool["tables"].cuda(), pool["lengths"].cuda()


def test_noalloc_entry_matches_the_workspace_entry_on_two_calls_in_a_row():
    lib = _capi.load()
    torch.cuda.set_device(0)
    # call 1 leaves multi-chunk partials, counters and a work list behind in the shared block;
    # call 2 is a different batch (other groups, other lengths, an empty row) on the same block.
    cases = [make_case(1, [1300, 40, 700], 5), make_case(2, [90, 2100], 7)]
    cases[1][4][3] = 0  # one empty row in the second batch
    for q, key, value, tables, lengths in cases:
        need = lib.rlt_verify_attention_workspace_bytes(q.shape[0], 16, 16, 128, 16, tables.shape[1])
        workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
        status, want = call_entry(lib, "rlt_verify_attention", q, key, value, tables, lengths, workspace)
        assert status == 0, _capi.last_error()
        status, got = call_entry(lib, "rlt_verify_attention_noalloc", q, key, value, tables, lengths)
        assert status == 0, _capi.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert bool(torch.isfinite(got.float()).all())
    assert torch.count_nonzero(got[3]) == 0


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
