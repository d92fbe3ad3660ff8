"""Sliding-window paged attention (`AttentionBackend.windowed`) against the reference's outputs and the oracle."""

import pytest
import torch

import vllm_rlt_b200 as rlt
from helpers import attention_tolerance
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_window_grid_of_the_reference(golden):
    # the grid of the reference's GPU test of its Triton kernel, its fp32 tolerances (tests/test_dory_gpu.py:75-93)
    kernel = rlt.B200PagedAttention()
    for case in golden("windowed.pt")["grid"]:
        key, value, q, tables = (case[n].cuda() for n in ("key", "value", "q", "tables"))
        for (window, length), want in case["out"].items():
            lengths = torch.tensor([length], dtype=torch.int32, device="cuda")
            got = kernel.windowed(q, key, value, tables, lengths, window)
            torch.testing.assert_close(got.cpu(), want, atol=2e-6, rtol=2e-5)
            if window >= length:     # the whole context is inside the window: the unwindowed entry agrees
                torch.testing.assert_close(got, kernel(q, key, value, tables, lengths), atol=2e-6, rtol=2e-5)


def test_ragged_batch_in_bf16(golden):
    case = golden("windowed.pt")["batched"]
    kernel = rlt.B200PagedAttention()
    tol = attention_tolerance(torch.bfloat16)
    args = [case[n].cuda() for n in ("q", "key", "value", "tables", "lengths")]
    for window, want in case["out"].items():
        got = kernel.windowed(*args, window)
        torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol, rtol=tol)
        assert not got[0].any()                                      # the row without context
        mine = oracle.paged_attention_windowed(case["q"], case["key"], case["value"], case["tables"], case["lengths"], window)
        torch.testing.assert_close(got.float().cpu(), mine.float(), atol=tol, rtol=tol)
    narrow, wide = kernel.windowed(*args, 5), kernel.windowed(*args, 200)
    assert torch.equal(narrow[:3], wide[:3]) and not torch.equal(narrow[3:], wide[3:])   # lengths 0, 1, 5 fit a window of 5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_layer_view_gqa_odd_head_size_and_graph_capture(dtype):
    # a layer view of a [blocks, layers, ...] pool, 6 query heads over 3 KV heads of 80, 8-token pages; replayed from a graph
    g = torch.Generator().manual_seed(5)
    pool = (torch.randn(2, 50, 3, 8, 3, 80, generator=g) * 0.5).to(dtype)
    key, value = pool[0][:, 1], pool[1][:, 1]
    lengths = torch.tensor([33, 8, 9, 64, 0], dtype=torch.int32)
    tables = torch.randperm(50, generator=g)[:40].view(5, 8).int()
    q = (torch.randn(5, 6, 80, generator=g) * 0.5).to(dtype)
    want = oracle.paged_attention_windowed(q, key, value, tables, lengths, 9)
    kernel = rlt.B200PagedAttention()
    device_pool = pool.cuda()
    args = (q.cuda(), device_pool[0][:, 1], device_pool[1][:, 1], tables.cuda(), lengths.cuda())
    got = kernel.windowed(*args, 9)
    tol = attention_tolerance(dtype)
    torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol, rtol=tol)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = kernel.windowed(*args, 9)
    args[4].fill_(0)                     # lengths live on the device: a replay sees the new ones
    graph.replay()
    torch.cuda.synchronize()
    assert not captured.any()


def test_misuse_raises_what_the_reference_raises():
    kernel = rlt.B200PagedAttention()
    q = torch.zeros(1, 2, 64, device="cuda")
    k = torch.zeros(2, 16, 2, 64, device="cuda")
    tables, lengths = torch.zeros(1, 2, dtype=torch.int32, device="cuda"), torch.ones(1, dtype=torch.int32, device="cuda")
    for window in (0, -3, True, 2.0, None):
        with pytest.raises(ValueError, match="window must be a positive integer"):      # kernels/paged_attention.py:53-54
            kernel.windowed(q, k, k, tables, lengths, window)
    with pytest.raises(ValueError, match="one block-table row"):
        kernel.windowed(q, k, k, tables, torch.ones(2, dtype=torch.int32, device="cuda"), 4)
    backend = rlt.create_backend("cuda", torch.float32, 64, 16)
    assert backend.capabilities.sliding_window
    assert backend.windowed(q, k, k, tables, lengths, 4).shape == q.shape
