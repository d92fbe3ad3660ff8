"""Builders shared by the tests: seeded paged KV pools and verification rounds."""

from __future__ import annotations

import torch


def make_pool(lengths_per_group, *, kv_heads, head_dim, block, dtype, seed, layers=1, layer=0,
              rows_per_group=1, row_lengths=None, extra_pages=2, scale=0.5, pad=-1, poison=True):
    """A paged pool where every group (request x plane) owns a random set of pages.

    lengths_per_group[g]: tokens stored for group g.  Each group contributes ``rows_per_group``
    query rows (or explicit ``row_lengths[g]``: list of visible lengths), all pointing at the
    group's block-table row.  Returns CPU tensors:
    key/value layer views, block_tables [rows, width], context_lengths [rows], group_of_row.

    ``poison``: every slot no group has stored a token in — behind a group's last token inside its last
    page, and the pages nobody owns — holds NaN, as a cache allocated with ``torch.empty`` may (the
    reference allocates its pools that way, core/kv_cache_manager.py:143-145).  No result may depend on them.
    """
    g = torch.Generator().manual_seed(seed)
    pages_per_group = [-(-n // block) for n in lengths_per_group]
    total_pages = sum(pages_per_group) + extra_pages
    shape = (total_pages, layers, block, kv_heads, head_dim)
    key = (torch.randn(shape, generator=g) * scale).to(dtype)
    value = (torch.randn(shape, generator=g) * scale).to(dtype)
    order = torch.randperm(total_pages, generator=g).tolist()
    width = max(pages_per_group + [1])
    tables, lengths, owner = [], [], []
    written = torch.zeros(total_pages, block, dtype=torch.bool)
    for gi, (n, pages) in enumerate(zip(lengths_per_group, pages_per_group)):
        ids = [order.pop() for _ in range(pages)]
        for index, page in enumerate(ids):
            written[page, : max(0, min(block, n - index * block))] = True
        row = ids + [pad] * (width - pages)
        visible = row_lengths[gi] if row_lengths is not None else [n] * rows_per_group
        for length in visible:
            tables.append(row)
            lengths.append(length)
            owner.append(gi)
    if poison:
        hole = ~written[:, None, :, None, None].expand_as(key)
        key.masked_fill_(hole, float("nan"))
        value.masked_fill_(hole, float("nan"))
    return dict(
        key=key[:, layer], value=value[:, layer], key_pool=key, value_pool=value,
        tables=torch.tensor(tables, dtype=torch.int32).reshape(len(tables), width),
        lengths=torch.tensor(lengths, dtype=torch.int32), owner=owner,
    )


def to_cuda_view(pool_tensor, layer):
    """Move a whole [pages, layers, ...] pool to the GPU and return one layer's strided view."""
    return pool_tensor.cuda()[:, layer]


def attention_tolerance(dtype):
    # bf16 / fp16: the tolerances the reference's own GPU tests use (tests/test_attention.py:54);
    # fp32: the 1e-5 relative bound of the task statement.
    return {torch.bfloat16: 2e-2, torch.float16: 2e-3, torch.float32: 1e-5}[dtype]
