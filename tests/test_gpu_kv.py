"""KV write and device rollback vs the CPU oracle and the reference's golden frontiers."""

import pytest
import torch

import vllm_rlt_b200 as rlt
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,block", [(16, 128, 16), (2, 7, 3), (4, 64, 16)])
def test_kv_write_matches_oracle_on_a_layer_strided_pool(dtype, heads, dim, block):
    g = torch.Generator().manual_seed(5)
    blocks, layers, layer, rows = 23, 3, 1, 11
    sentinel = 7.0
    pool_k = torch.full((blocks, layers, block, heads, dim), sentinel).to(dtype)
    pool_v = torch.full((blocks, layers, block, heads, dim), -sentinel).to(dtype)
    k = torch.randn(rows, heads, dim, generator=g).to(dtype)
    v = torch.randn(rows, heads, dim, generator=g).to(dtype)
    slots = torch.randperm(blocks * block, generator=g)[:rows]
    write_blocks, write_offsets = slots // block, slots % block
    mask = torch.tensor([True, True, False, True, True, True, True, False, True, True, True])
    active = torch.tensor(9, dtype=torch.int32)
    want_k, want_v = pool_k.clone(), pool_v.clone()
    oracle.kv_write(want_k[:, layer], want_v[:, layer], k, v, write_blocks, write_offsets, mask, active)
    got_k, got_v = pool_k.cuda(), pool_v.cuda()
    # padding rows carry addresses that must never be loaded
    bad_blocks = write_blocks.clone()
    bad_blocks[2] = 10**12
    bad_blocks[9:] = -5
    rlt.kv_write(got_k[:, layer], got_v[:, layer], k.cuda(), v.cuda(), bad_blocks.cuda(),
                 write_offsets.cuda(), mask.cuda(), active.cuda())
    assert torch.equal(got_k.cpu().view(torch.uint8), want_k.view(torch.uint8))
    assert torch.equal(got_v.cpu().view(torch.uint8), want_v.view(torch.uint8))
    # other layers and unwritten slots keep their sentinel bytes
    assert torch.equal(got_k[:, 0].cpu(), pool_k[:, 0]) and torch.equal(got_k[:, 2].cpu(), pool_k[:, 2])


def test_kv_write_without_mask_and_empty_batch():
    cache_k = torch.zeros(4, 16, 2, 8, device="cuda")
    cache_v = torch.zeros_like(cache_k)
    k = torch.randn(3, 2, 8, device="cuda")
    blocks = torch.tensor([3, 0, 2], device="cuda")
    offsets = torch.tensor([15, 0, 7], device="cuda")
    rlt.kv_write(cache_k, cache_v, k, -k, blocks, offsets)
    assert torch.equal(cache_k[blocks, offsets], k) and torch.equal(cache_v[blocks, offsets], -k)
    empty = torch.empty(0, 2, 8, device="cuda")
    rlt.kv_write(cache_k, cache_v, empty, empty, blocks[:0], offsets[:0])
    with pytest.raises(ValueError, match="int64"):
        rlt.kv_write(cache_k, cache_v, k, k, blocks.int(), offsets)


def test_rollback_matches_reference_frontiers(golden):
    for case in golden("rollback.pt"):
        if case.get("shared"):
            tables = case["tables"][None].contiguous().cuda()
            for frontier, want in ((case["refused_frontier"], 4), (case["allowed_frontier"], 0)):
                out = rlt.rollback(torch.tensor([0]).cuda(), torch.tensor([frontier]).cuda(), tables,
                                   case["block"], refcounts=case["refcounts"].cuda())
                assert int(out.status[0]) == want
            continue
        tables = case["tables"][None].contiguous().cuda()
        prefix = case["before"][None].clone().long().contiguous().cuda()
        out = rlt.rollback(torch.tensor([case["start"]]).cuda(), torch.tensor([case["emitted"]]).cuda(),
                           tables, case["block"], written_prefix=prefix)
        assert int(out.status[0]) == 0
        assert int(out.frontier[0]) == case["frontier"]
        assert torch.equal(prefix[0].cpu(), case["after"].long())
        assert int(out.context_lengths[0]) == case["context_length"]
        assert int(out.write_offsets[0]) == case["write_offset"]
        assert torch.equal(out.write_blocks[0].cpu(), case["write_blocks"])


def test_rollback_batch_matches_oracle_bit_for_bit():
    g = torch.Generator().manual_seed(9)
    n, planes, width, layers, block = 37, 4, 40, 24, 16
    tables = torch.randint(0, 5000, (n, planes, width), generator=g, dtype=torch.int32)
    starts = torch.randint(0, width * block - 8, (n,), generator=g)
    emitted = torch.randint(1, 6, (n,), generator=g)
    refcounts = (torch.rand(5000, generator=g) < 0.01).int() + 1
    pages_used = torch.randint(1, width + 1, (n,), generator=g, dtype=torch.int32)
    prefix = torch.randint(0, width * block, (n, planes, layers), generator=g)
    want_prefix = prefix.clone()
    want = oracle.rollback(starts, emitted, tables, block, pages_used, refcounts, want_prefix)
    got_prefix = prefix.clone().cuda()
    got = rlt.rollback(starts.cuda(), emitted.cuda(), tables.cuda(), block, pages_used=pages_used.cuda(),
                       refcounts=refcounts.cuda(), written_prefix=got_prefix)
    ok = want[4] == 0
    assert torch.equal(got.status.cpu(), want[4]) and 0 < int(ok.sum()) < n
    assert torch.equal(got.frontier.cpu(), want[0])
    assert torch.equal(got.context_lengths.cpu()[ok], want[1][ok])
    assert torch.equal(got.write_blocks.cpu()[ok], want[2][ok])
    assert torch.equal(got.write_offsets.cpu()[ok], want[3][ok])
    assert torch.equal(got_prefix.cpu(), want_prefix)
    assert torch.equal(tables, tables.clone())  # tables are inputs only


def test_finalize_tokens_match_the_reference_and_the_oracle(golden):
    for case in golden("finalize.pt"):
        key, value = case["key_before"].cuda(), case["value_before"].cuda()
        rlt.finalize_tokens(key, value, case["tables"].cuda(), case["slots"].cuda(), case["depths"].cuda(),
                            case["positions"].cuda())
        assert torch.equal(key.cpu().view(torch.uint8), case["key_after"].view(torch.uint8))
        assert torch.equal(value.cpu().view(torch.uint8), case["value_after"].view(torch.uint8))
    # a larger seeded case against the oracle: Ouro-shaped rows, every exit depth
    g = torch.Generator().manual_seed(4)
    slots_n, planes, width, layers, block = 9, 4, 6, 24, 16
    tables = torch.randperm(slots_n * planes * width, generator=g).int().view(slots_n, planes, width)
    pool = (slots_n * planes * width, layers, block, 16, 128)
    key = torch.randn(pool, generator=g).bfloat16()
    value = torch.randn(pool, generator=g).bfloat16()
    slots = torch.arange(slots_n)
    depths = torch.tensor([0, 1, 2, 3, 0, 1, 2, 0, 1])
    positions = torch.randint(0, width * block, (slots_n,), generator=g)
    want_k, want_v = key.clone(), value.clone()
    oracle.finalize_tokens(want_k, want_v, tables, slots, depths, positions)
    got_k, got_v = key.cuda(), value.cuda()
    rlt.finalize_tokens(got_k, got_v, tables.cuda(), slots.cuda(), depths.cuda(), positions.cuda())
    assert torch.equal(got_k.cpu().view(torch.int16), want_k.view(torch.int16))
    assert torch.equal(got_v.cpu().view(torch.int16), want_v.view(torch.int16))
    assert not torch.equal(want_k, key)


def test_rollback_to_the_last_token_of_a_full_allocation_is_valid():
    # truncate_suffix accepts 0 <= frontier <= max_tokens (core/kv_cache_manager.py:340-342 of the reference):
    # a request that filled its pages exactly is rolled back like any other, only its next page does not exist
    planes, width, block, layers = 2, 3, 16, 2
    tables = torch.arange(2 * planes * width, dtype=torch.int32).view(2, planes, width)
    starts, emitted = torch.tensor([width * block - 3, width * block - 3]), torch.tensor([3, 4])
    prefix = torch.full((2, planes, layers), width * block + 5)
    want_prefix = prefix.clone()
    want = oracle.rollback(starts, emitted, tables, block, None, None, want_prefix)
    got_prefix = prefix.clone().cuda()
    got = rlt.rollback(starts.cuda(), emitted.cuda(), tables.cuda(), block, written_prefix=got_prefix)
    assert got.status.tolist() == want[4].tolist() == [0, 5]       # exactly full is fine, one beyond is refused
    assert got.frontier.tolist() == [width * block, width * block + 1]
    assert got.context_lengths.tolist()[0] == width * block + 1 and got.write_blocks.tolist()[0] == [-1, -1]
    assert torch.equal(got.write_blocks.cpu()[0], want[2][0])
    assert torch.equal(got_prefix.cpu(), want_prefix) and int(got_prefix[0].max()) == width * block
    assert int(got_prefix[1].max()) == width * block + 5             # the refused request is untouched
