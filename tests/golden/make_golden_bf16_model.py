"""Golden hidden states and logits of a bf16 looped LM with Ouro-shaped heads, from the vllm-rlt reference.

    PYTHONPATH=<reference checkout>:<reference checkout>/tests python tests/golden/make_golden_bf16_model.py

The reference's own Torch execution (CPU, bfloat16 weights and activations, its paged KV cache with
16-token pages and `torch_paged_attention`) runs every token of three seeded sequences one position
at a time through all four recurrent loops — the serial replay its tests use as the oracle for
speculative rounds (tests/test_speculative.py:134-150 there).  Stored in `bf16_model.pt`: the model
shape and weight seed (the weights themselves are rebuilt from `seeded_parameter`, as in
`make_golden_decode.py`), the sequences, the normalised hidden state of every position after every
loop depth, and the LM-head logits of the final depth.

The heads are 2 x 128 with 16-token pages, so the GPU side of the comparison goes through the tiled
TMA / tensor-core verify kernel and the tcgen05 prompt kernels rather than the shape-generic one.
"""

from __future__ import annotations

from pathlib import Path

import torch

from make_golden_decode import build
from vllm_rlt import CacheConfig
from vllm_rlt.engine.llm_engine import LLMEngine
from vllm_rlt.models import OuroConfig

HERE = Path(__file__).resolve().parent
torch.set_num_threads(4)


def main():
    config = OuroConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=2, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
                        rope_theta=10000.0, total_ut_steps=4, max_position_embeddings=256,
                        bos_token_id=0, eos_token_id=0)
    seed, block = 21, 16
    model = build(config, seed).to(torch.bfloat16)
    g = torch.Generator().manual_seed(77)
    sequences = [torch.randint(1, config.vocab_size, (n,), generator=g).tolist() for n in (45, 8, 22)]
    cache = LLMEngine(model, cache_config=CacheConfig(64, block), attention_backend="torch").cache_manager
    hidden_states, logits = [], []
    with torch.inference_mode():
        for index, tokens in enumerate(sequences):
            rid = f"s{index}"
            assert cache.allocate(rid, len(tokens) + 1)
            per_depth = [[] for _ in range(config.total_ut_steps)]
            rows = []
            for position, token in enumerate(tokens):
                h = model.prelude(torch.tensor([token]))
                for depth in range(config.total_ut_steps):
                    h, _ = model.recurrent(h, [rid], [depth], [position], cache)
                    per_depth[depth].append(h[0].clone())
                rows.append(model.coda(h)[0].clone())
            hidden_states.append(torch.stack([torch.stack(d) for d in per_depth]))   # [depths, positions, hidden]
            logits.append(torch.stack(rows))                                          # [positions, vocab]
    fields = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "total_ut_steps", "initializer_range")
    torch.save(dict(config={f: getattr(config, f) for f in fields}, seed=seed, block=block, sequences=sequences,
                    hidden=hidden_states, logits=logits), HERE / "bf16_model.pt")
    for tokens, h, l in zip(sequences, hidden_states, logits):
        print(len(tokens), tuple(h.shape), tuple(l.shape), float(l.float().abs().max()))


if __name__ == "__main__":
    main()
