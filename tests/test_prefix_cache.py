"""Prefix index and shared page tables (host logic; the rules of the reference's KVCacheManager,
tests/test_kv_cache.py:177-198 and tests/test_prefix_growth.py:27-60 there)."""

from types import SimpleNamespace

import torch

from vllm_rlt_b200.decoder import PagedKV
from vllm_rlt_b200.prefix_cache import PrefixIndex, page_keys


def test_keys_chain_over_complete_pages_only():
    a = list(page_keys([1, 2, 3, 4, 5], 2))
    assert len(a) == 2                                   # the fifth token does not fill a page
    assert a[0] == list(page_keys([1, 2], 2))[0]
    assert a[1] != list(page_keys([9, 9, 3, 4], 2))[1]   # same page tokens, different history


def test_lookup_leaves_the_last_token_and_stops_at_the_first_miss():
    index = PrefixIndex(2)
    tables = [[10, 11, 12], [20, 21, 22]]                 # two depth planes, three pages
    assert index.publish([1, 2, 3, 4, 5], 5, tables) == 2
    assert index.lookup([1, 2, 3, 4, 5]) == ((10, 20), (11, 21))
    assert index.lookup([1, 2, 3, 4]) == ((10, 20),)      # tokens[:-1] holds one complete page
    assert len(index.lookup([1, 2, 9, 4, 5])) == 1        # a different continuation keeps the first page
    assert index.lookup([7, 2, 3, 4, 5]) == ()
    assert index.publish([1, 2, 3, 4, 5], 5, [[30, 31, 32], [40, 41, 42]]) == 0   # already indexed
    # a prompt that is a multiple of the page still recomputes its last token
    index.publish([1, 2, 3, 4], 4, tables)
    assert len(index.lookup([1, 2, 3, 4])) == 1


def test_reference_counts():
    index = PrefixIndex(2)
    index.own([10, 11, 12])
    index.publish([1, 2, 3, 4, 5], 5, [[10, 11, 12]])
    assert index.refs == {10: 2, 11: 2, 12: 1}            # owner + index; the last page is not indexed
    hit = index.lookup([1, 2, 3, 4, 9])
    index.claim(hit)
    assert index.refs[10] == 3 and index.refs[11] == 3
    assert index.shared(10) and not index.shared(12)
    assert (index.queries, index.hit_tokens) == (1, 4)


def fake_model(planes=2):
    config = SimpleNamespace(total_ut_steps=planes, num_hidden_layers=1, num_key_value_heads=1, head_dim=8)
    return SimpleNamespace(config=config, device="cpu", dtype=torch.float32)


def test_page_tables_share_the_indexed_prefix_on_every_plane():
    g = torch.Generator().manual_seed(0)
    base = torch.randint(1, 100, (40,), generator=g).tolist()
    prompts = [base, base[:33] + [101, 102, 103], list(base), [5, 6, 7]]
    capacities = [len(p) + 8 for p in prompts]
    plain = PagedKV.allocate(fake_model(), capacities, 16)
    kv = PagedKV.allocate(fake_model(), capacities, 16, prompts=prompts)
    assert plain.shared_tokens == [0, 0, 0, 0]
    assert kv.shared_tokens == [0, 32, 32, 0]             # two complete pages of prompt[:-1]
    assert kv.key.shape[0] == plain.key.shape[0] - 2 * 2 * 2
    t = kv.tables
    for follower in (1, 2):
        assert torch.equal(t[follower, :, :2], t[0, :, :2])
        assert not torch.equal(t[follower, :, 2], t[0, :, 2])
    used = t[t >= 0]
    assert used.unique().numel() == kv.key.shape[0]        # every page of the pool is mapped
    shared = set(t[0, :, :2].reshape(-1).tolist())
    assert all(kv.prefix_index.refs[b] == 4 for b in shared)          # owner + index + two followers
    assert all(kv.prefix_index.refs[b] <= 2 for b in set(used.tolist()) - shared)
    assert kv.prefix_index.hit_tokens == 64


def test_matching_an_entry_makes_it_the_most_recent():
    index = PrefixIndex(2)
    index.publish([1, 2, 3], 3, [[10, 11]])
    index.publish([7, 8, 9], 3, [[20, 21]])
    first, second = list(page_keys([1, 2], 2))[0], list(page_keys([7, 8], 2))[0]
    assert index.least_recent() == first
    index.lookup([1, 2, 5])
    assert index.least_recent() == second
    assert PrefixIndex(2).least_recent() is None
