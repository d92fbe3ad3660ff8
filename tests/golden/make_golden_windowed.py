"""Golden vectors of sliding-window paged attention, from the vllm-rlt reference.

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_windowed.py

`torch_paged_attention_windowed` (vllm_rlt/kernels/paged_attention.py:39-70) on the grid of the
reference's own GPU test of its Triton kernel (tests/test_dory_gpu.py:75-93: fp32, 16-token pages,
4 query heads over 2 KV heads, head_dim 8 / 128 / 256, windows 1 / 3 / 16 / 64, lengths
1 / 7 / 63 / 64 / 65 over 8 pages), one set of K / V / Q per head size; plus one batched bf16 case with
ragged lengths (an empty row, rows shorter than, equal to and longer than the window) and pages in
random order, through `KVCacheManager.attend(..., window=...)`'s kernel call shape.
Stored in `windowed.pt`: the inputs and, per (window, length), the reference's output.
"""

from __future__ import annotations

from pathlib import Path

import torch

from vllm_rlt.kernels.paged_attention import torch_paged_attention_windowed

HERE = Path(__file__).resolve().parent
torch.set_num_threads(1)


def main():
    grid = []
    for head_dim in (8, 128, 256):
        g = torch.Generator().manual_seed(head_dim)
        keys = torch.randn(8, 16, 2, head_dim, generator=g)
        values = torch.randn(8, 16, 2, head_dim, generator=g)
        query = torch.randn(1, 4, head_dim, generator=g)
        tables = torch.arange(8, dtype=torch.int32)[None, :]
        outputs = {}
        for window in (1, 3, 16, 64):
            for length in (1, 7, 63, 64, 65):
                lengths = torch.tensor([length], dtype=torch.int32)
                outputs[(window, length)] = torch_paged_attention_windowed(query, keys, values, tables, lengths, window)
        grid.append(dict(head_dim=head_dim, key=keys, value=values, q=query, tables=tables, out=outputs))
    g = torch.Generator().manual_seed(99)
    lengths = torch.tensor([0, 1, 5, 6, 40, 77], dtype=torch.int32)
    keys = (torch.randn(40, 16, 2, 64, generator=g) * 0.5).bfloat16()
    values = (torch.randn(40, 16, 2, 64, generator=g) * 0.5).bfloat16()
    query = (torch.randn(6, 8, 64, generator=g) * 0.5).bfloat16()
    tables = torch.randperm(40, generator=g)[:30].view(6, 5).int()
    batched = dict(key=keys, value=values, q=query, tables=tables, lengths=lengths,
                   out={w: torch_paged_attention_windowed(query, keys, values, tables, lengths, w) for w in (5, 16, 200)})
    torch.save(dict(grid=grid, batched=batched), HERE / "windowed.pt")
    print("cases", sum(len(c["out"]) for c in grid) + len(batched["out"]))


if __name__ == "__main__":
    main()
