"""Packed causal prefill kernel vs the reference's outputs, the CPU oracle and the verify kernel."""

import pytest
import torch

import vllm_rlt_b200 as rlt
from helpers import attention_tolerance
from oracle import oracle

pytestmark = pytest.mark.gpu


def check(got, want, dtype):
    tol = attention_tolerance(dtype)
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), rtol=tol, atol=tol)


def make_case(new, context, *, q_heads, kv_heads, dtype, seed, layers=1, layer=0, value_first=False):
    """Sequences with `new[s]` query tokens on top of `context[s] - new[s]` cached ones."""
    g = torch.Generator().manual_seed(seed)
    block, dim = 16, 128
    pages = [-(-c // block) for c in context]
    total = sum(pages) + 3
    shape = (total, layers, block, kv_heads, dim)
    both = (torch.randn((2,) + shape, generator=g) * 0.5).to(dtype)       # one allocation: the address order is ours
    key, value = (both[1], both[0]) if value_first else (both[0], both[1])
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages)
    tables = torch.full((len(new), width), -1, dtype=torch.int32)
    written = torch.zeros(total, block, dtype=torch.bool)
    for s, n in enumerate(pages):
        ids = [order.pop() for _ in range(n)]
        tables[s, :n] = torch.tensor(ids, dtype=torch.int32)
        for index, page in enumerate(ids):
            written[page, : max(0, min(block, context[s] - index * block))] = True
    # slots nobody stored a token in hold NaN, as a pool allocated with torch.empty may: no result may depend on them
    both.masked_fill_(~written[None, :, None, :, None, None].expand_as(both), float("nan"))
    q = (torch.randn(sum(new), q_heads, dim, generator=g) * 0.5).to(dtype)
    cu = torch.tensor([0] + torch.tensor(new).cumsum(0).tolist(), dtype=torch.int32)
    return dict(q=q, both=both, value_first=value_first, layer=layer, tables=tables,
                lengths=torch.tensor(context, dtype=torch.int32), cu=cu,
                key=key[:, layer], value=value[:, layer])


def run_prefill(kernel, case, max_new):
    both = case["both"].cuda()
    key, value = (both[1], both[0]) if case["value_first"] else (both[0], both[1])
    out = kernel.prefill(case["q"].cuda(), key[:, case["layer"]], value[:, case["layer"]], case["tables"].cuda(),
                         case["lengths"].cuda(), case["cu"].cuda(), max_new)
    torch.cuda.synchronize()
    return out


def test_prefill_of_the_reference(golden):
    case = golden("prefill.pt")
    kernel = rlt.B200PagedAttention()
    out = kernel.prefill(case["q"].cuda(), case["key"].cuda(), case["value"].cuda(), case["tables"].cuda(),
                         case["lengths"].cuda(), case["cu_seqlens_q"].cuda(), 129)
    check(out, case["out"], torch.bfloat16)


@pytest.fixture(params=["pair", "umma", "mma"])
def forced_kernel(request, monkeypatch):
    """Each of the three prefill kernels in turn (the library reads the variable at every call)."""
    monkeypatch.setenv("RLT_PREFILL_KERNEL", request.param)
    return request.param


def test_each_prefill_kernel_on_tile_edges_and_long_contexts(forced_kernel):
    # 128 / 256-row tile edges, a second tile with one row, contexts that wrap the stage ring
    new = [1, 127, 128, 129, 255, 256, 257, 700, 33, 5]
    context = [1, 127, 128, 129, 255, 256, 900, 700, 2000, 1234]
    for dtype in (torch.bfloat16, torch.float16):
        case = make_case(new, context, q_heads=4, kv_heads=2, dtype=dtype, seed=11, layers=2, layer=1)
        got = run_prefill(rlt.B200PagedAttention(), case, max(new))
        want = oracle.paged_attention(case["q"], case["key"], case["value"], case["tables"].clamp_min(0),
                                      case["lengths"], case["cu"])
        check(got, want, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("q_heads,kv_heads", [(4, 4), (4, 2), (8, 1)])
@pytest.mark.parametrize("value_first", [False, True])
def test_prefill_matches_oracle_and_the_verify_kernel(dtype, q_heads, kv_heads, value_first):
    # tile edges (63, 64, 65 queries), a single token, a long prompt, cached prefixes shorter and
    # longer than the new tokens, a prefix that is not a multiple of the page or of the key tile
    new = [1, 63, 64, 65, 300, 17, 128, 40]
    context = [1, 63, 64, 65, 300, 1000, 130, 777]
    case = make_case(new, context, q_heads=q_heads, kv_heads=kv_heads, dtype=dtype, seed=q_heads + kv_heads,
                     layers=2, layer=1, value_first=value_first)
    kernel = rlt.B200PagedAttention()
    got = run_prefill(kernel, case, max(new))
    want = oracle.paged_attention(case["q"], case["key"], case["value"], case["tables"].clamp_min(0), case["lengths"],
                                  case["cu"])
    check(got, want, dtype)
    grouped = run_prefill(kernel, case, 0)          # the same rows through the grouped verify kernel
    check(got, grouped, dtype)
    assert not torch.equal(got, grouped)              # two kernels (no split-KV merge in the prefill one)


def test_pair_kernel_on_more_ragged_tiles_than_sms(monkeypatch):
    # several waves of CTAs (256-row tiles x heads), ragged: full pairs, lone first tiles, second tiles of a few
    # rows, an empty sequence.  All rows against the mma.sync kernel, a sample of sequences against the oracle.
    g = torch.Generator().manual_seed(23)
    new = torch.randint(1, 700, (90,), generator=g).tolist()
    new[3], new[4], new[5], new[40] = 0, 256, 257, 1
    context = [n + int(torch.randint(0, 300, (1,), generator=g)) for n in new]
    context = [max(c, 1) for c in context]
    case = make_case(new, context, q_heads=4, kv_heads=2, dtype=torch.bfloat16, seed=29)
    kernel = rlt.B200PagedAttention()
    monkeypatch.setenv("RLT_PREFILL_KERNEL", "pair")
    got = run_prefill(kernel, case, max(new))
    again = run_prefill(kernel, case, max(new))
    assert torch.equal(got, again)
    monkeypatch.setenv("RLT_PREFILL_KERNEL", "mma")
    check(got, run_prefill(kernel, case, max(new)), torch.bfloat16)
    cu = case["cu"].tolist()
    longest = max(range(len(new)), key=lambda s: context[s])
    for s in (0, 4, 5, 40, 89, longest):
        rows = slice(cu[s], cu[s + 1])
        want = oracle.paged_attention(case["q"][rows], case["key"], case["value"], case["tables"][s:s + 1].clamp_min(0),
                                      case["lengths"][s:s + 1], torch.tensor([0, new[s]], dtype=torch.int32))
        check(got[rows], want, torch.bfloat16)


def test_prefill_handles_many_sequences_and_empty_ones():
    g = torch.Generator().manual_seed(3)
    new = torch.randint(0, 90, (1500,), generator=g).tolist()      # more sequences than one plan pass covers
    new[7] = 0
    context = [n + int(torch.randint(0, 40, (1,), generator=g)) for n in new]
    context = [max(c, 1) for c in context]
    case = make_case(new, context, q_heads=2, kv_heads=2, dtype=torch.bfloat16, seed=5)
    kernel = rlt.B200PagedAttention()
    got = run_prefill(kernel, case, 89)
    want = oracle.paged_attention(case["q"], case["key"], case["value"], case["tables"].clamp_min(0), case["lengths"],
                                  case["cu"])
    check(got, want, torch.bfloat16)


def test_prefill_of_other_shapes_falls_back_to_the_general_kernels():
    # fp32 / head_dim 64 is outside the tiled kernels: same call, same answer from the generic kernel
    g = torch.Generator().manual_seed(9)
    block, dim, heads = 16, 64, 2
    new, context = [40, 33], [40, 50]
    pages = [-(-c // block) for c in context]
    key = torch.randn(sum(pages), block, heads, dim, generator=g)
    value = torch.randn(sum(pages), block, heads, dim, generator=g)
    tables = torch.tensor([[0, 1, 2, 0], [3, 4, 5, 6]], dtype=torch.int32)
    q = torch.randn(sum(new), heads, dim, generator=g)
    cu = torch.tensor([0, 40, 73], dtype=torch.int32)
    lengths = torch.tensor(context, dtype=torch.int32)
    got = rlt.B200PagedAttention().prefill(q.cuda(), key.cuda(), value.cuda(), tables.cuda(), lengths.cuda(), cu.cuda(), 40)
    want = oracle.paged_attention(q, key, value, tables, lengths, cu)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)
