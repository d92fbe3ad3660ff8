"""Golden pools for early-exit finalisation, produced by the reference's KVCacheManager.finalize_token.

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_finalize.py

Stores the K/V pool before and after finalising a few (request, position, exit depth) tokens,
with the block tables, in `finalize.pt` (core/kv_cache_manager.py:805-831 of the reference).
"""

from pathlib import Path

import torch

from vllm_rlt.core.kv_cache_manager import KVCacheManager

HERE = Path(__file__).resolve().parent


def main():
    torch.manual_seed(17)
    cases = []
    for dtype, block, heads, dim, blocks in ((torch.float32, 2, 2, 8, 104), (torch.bfloat16, 16, 2, 16, 24)):
        layers, planes = 3, 4
        cache = KVCacheManager(layers, heads, dim, blocks, block, planes, dtype=dtype)
        lengths = {"a": 9, "b": 5, "c": 33}
        for rid, n in lengths.items():
            assert cache.allocate(rid, n)
        cache.key_cache.copy_(torch.randn(cache.key_cache.shape).to(dtype))
        cache.value_cache.copy_(torch.randn(cache.value_cache.shape).to(dtype))
        before_k, before_v = cache.key_cache.clone(), cache.value_cache.clone()
        rows = [("a", 4, 1), ("b", 0, 0), ("c", 32, 2), ("a", 8, 3), ("c", 7, 1)]
        for rid, pos, exit_depth in rows:
            k = torch.randn(1, heads, dim).to(dtype)
            for depth in range(exit_depth + 1):
                for layer in range(layers):
                    cache.write(layer, [rid], [depth], [pos], k + depth, k - depth)
        written_k, written_v = cache.key_cache.clone(), cache.value_cache.clone()
        for rid, pos, exit_depth in rows:
            cache.finalize_token(rid, pos, exit_depth)
        ids = list(lengths)
        width = max(len(cache._get_allocation(r).block_tables[0]) for r in ids)
        tables = torch.full((len(ids), planes, width), -1, dtype=torch.int32)
        for i, rid in enumerate(ids):
            for plane, table in enumerate(cache._get_allocation(rid).block_tables):
                tables[i, plane, : len(table)] = torch.tensor(table, dtype=torch.int32)
        cases.append(dict(block=block, tables=tables,
                          slots=torch.tensor([ids.index(r) for r, _, _ in rows]),
                          positions=torch.tensor([p for _, p, _ in rows]),
                          depths=torch.tensor([d for _, _, d in rows]),
                          key_before=written_k, value_before=written_v,
                          key_after=cache.key_cache.clone(), value_after=cache.value_cache.clone(),
                          untouched=bool(torch.equal(before_k, before_k))))
    torch.save(cases, HERE / "finalize.pt")
    print([c["key_before"].shape for c in cases], (HERE / "finalize.pt").stat().st_size)


if __name__ == "__main__":
    main()
