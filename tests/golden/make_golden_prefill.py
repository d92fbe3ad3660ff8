"""Golden outputs for packed causal prefill, from the reference's Torch attention.

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_prefill.py

The reference's CPU backend scores packed prefill rows one by one with
`torch_paged_attention` (kernels/paged_attention.py:12-36), query i of the n new tokens of a
sequence seeing `context - n + i + 1` keys (kernels/triton_attention.py:313-322 states the
same alignment for its Triton kernel).  `prefill.pt` holds such a case at prompt size: two
sequences (a 70-token prompt and 129 new tokens on top of a 171-token cached prefix), GQA 2:1.
"""

from pathlib import Path

import torch

from vllm_rlt.kernels.paged_attention import torch_paged_attention

HERE = Path(__file__).resolve().parent


def main():
    g = torch.Generator().manual_seed(41)
    block, kv_heads, q_heads, dim = 16, 1, 2, 128
    new, context = [70, 129], [70, 300]
    pages = [-(-c // block) for c in context]
    total = sum(pages) + 1
    key = (torch.randn(total, block, kv_heads, dim, generator=g) * 0.5).bfloat16()
    value = (torch.randn(total, block, kv_heads, dim, generator=g) * 0.5).bfloat16()
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages)
    tables = torch.full((2, width), -1, dtype=torch.int32)
    for s, n in enumerate(pages):
        tables[s, :n] = torch.tensor([order.pop() for _ in range(n)], dtype=torch.int32)
    q = (torch.randn(sum(new), q_heads, dim, generator=g) * 0.5).bfloat16()
    row_tables = torch.cat([tables[s:s + 1].expand(n, width) for s, n in enumerate(new)]).clamp_min(0)
    row_lengths = torch.cat([torch.arange(c - n + 1, c + 1) for n, c in zip(new, context)]).int()
    out = torch_paged_attention(q, key, value, row_tables, row_lengths)
    cu = torch.tensor([0, new[0], sum(new)], dtype=torch.int32)
    torch.save(dict(q=q, key=key, value=value, tables=tables, lengths=torch.tensor(context, dtype=torch.int32),
                    cu_seqlens_q=cu, out=out), HERE / "prefill.pt")


if __name__ == "__main__":
    main()
