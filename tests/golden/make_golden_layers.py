"""Golden outputs of the elementwise layer pieces around the attention call, from the reference.

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_layers.py

`layers.pt` holds, per dtype: RMSNorm outputs and the sandwich residual flow of
OuroDecoderLayer.forward (layers/normalization.py:20-23, models/ouro.py:217-221 of the
reference), and apply_rotary_pos_emb on q, k with RotaryEmbedding's cos / sin
(layers/rotary_embedding.py:8-64).
"""

from pathlib import Path

import torch

from vllm_rlt.layers.normalization import RMSNorm
from vllm_rlt.layers.rotary_embedding import RotaryEmbedding, apply_rotary_pos_emb

HERE = Path(__file__).resolve().parent


def main():
    g = torch.Generator().manual_seed(23)
    out = dict(norm=[], rope=[])
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for rows, hidden, scale in ((4, 256, 1.0), (1, 2048, 4.0), (2, 100, 0.01)):
            first, second = RMSNorm(hidden, eps=1e-6), RMSNorm(hidden, eps=1e-6)
            with torch.no_grad():
                first.weight.copy_(1 + 0.2 * torch.randn(hidden, generator=g))
                second.weight.copy_(1 + 0.2 * torch.randn(hidden, generator=g))
            first, second = first.to(dtype), second.to(dtype)
            x = (torch.randn(rows, hidden, generator=g) * scale).to(dtype)
            residual = torch.randn(rows, hidden, generator=g).to(dtype)
            with torch.no_grad():
                plain = first(x)
                total = residual + first(x)            # hidden + input_layernorm_2(attention)
                following = second(total)              # post_attention_layernorm(hidden)
            out["norm"].append(dict(x=x, residual=residual, weight=first.weight.detach().clone(),
                                    weight2=second.weight.detach().clone(), eps=1e-6, plain=plain, total=total,
                                    following=following))
        for rows, q_heads, kv_heads, dim, theta in ((5, 2, 2, 64, 10000.0), (2, 16, 16, 128, 1_000_000.0),
                                                    (3, 4, 2, 32, 10000.0)):
            rotary = RotaryEmbedding(head_dim=dim, rope_theta=theta)
            q = torch.randn(rows, q_heads, dim, generator=g).to(dtype)
            k = torch.randn(rows, kv_heads, dim, generator=g).to(dtype)
            positions = torch.randint(0, 20000, (rows,), generator=g)
            cos, sin = rotary(q, positions)
            q_rot, k_rot = apply_rotary_pos_emb(q, k, cos, sin)
            out["rope"].append(dict(q=q, k=k, positions=positions, theta=theta, cos=cos.squeeze(1), sin=sin.squeeze(1),
                                    q_rot=q_rot, k_rot=k_rot))
    torch.save(out, HERE / "layers.pt")


if __name__ == "__main__":
    main()
