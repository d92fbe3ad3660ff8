"""Golden token sequences of self-speculative decoding, produced by the vllm-rlt reference engine.

    PYTHONPATH=<reference checkout>:<reference checkout>/tests python tests/golden/make_golden_decode.py

For each case the reference's Torch execution (CPU, fp32) decodes the same seeded prompts twice:
natively (one token per step through all loops) and with block self-speculation
(`SpeculativeConfig(k, draft_loops, target_loops)`).  Both token lists and the speculative
counters are stored in `decode.pt`; the weights are NOT stored — every parameter is overwritten
with `seeded_parameter(name, shape, seed)` below (a documented, order-independent rule that
`vllm_rlt_b200.looped_lm.seeded_state_dict` repeats), so the test rebuilds the same model.

Cases: the reference's own tiny test architecture (GQA 4/2 heads of dim 8, block size 2) and
the small CPU-runnable configuration (2 layers, hidden 256, 4 x 64 MHA, FFN 688, vocab 1024, 4 loops, 4 prompts x 32
tokens, 64 generated, k = 4 from depth 2 verified at depth 4, block size 16).
"""

from __future__ import annotations

import hashlib
from pathlib import Path

import torch

from helpers import LocalLLM
from vllm_rlt import CacheConfig, SamplingParams, SpeculativeConfig
from vllm_rlt.models import OuroConfig, OuroForCausalLM

HERE = Path(__file__).resolve().parent
torch.set_num_threads(1)


def seeded_parameter(name: str, shape, seed: int, std: float) -> torch.Tensor:
    """N(0, std) values for one named parameter from a generator seeded by (seed, name);
    norm weights are ones and biases zeros."""
    if name.endswith("norm.weight") or "layernorm" in name:
        return torch.ones(shape)
    if name.endswith(".bias"):
        return torch.zeros(shape)
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    generator = torch.Generator().manual_seed(int.from_bytes(digest[:7], "little"))
    return torch.randn(shape, generator=generator) * std


def build(config: OuroConfig, seed: int) -> OuroForCausalLM:
    model = OuroForCausalLM(config)
    state = {name: seeded_parameter(name, tuple(p.shape), seed, config.initializer_range)
             for name, p in model.state_dict().items()}
    model.load_state_dict(state, strict=True)
    return model


def run_case(config: OuroConfig, seed: int, prompts, max_tokens: int, k: int, draft: int, target: int,
             blocks: int, block: int):
    model = build(config, seed)
    params = SamplingParams(max_tokens=max_tokens, ignore_eos=True)
    native = LocalLLM(model, cache_config=CacheConfig(blocks, block)).generate(prompts, params)
    llm = LocalLLM(model, speculative_config=SpeculativeConfig(k, draft_loops=draft, target_loops=target),
                   cache_config=CacheConfig(blocks, block))
    speculative = llm.generate(prompts, params)
    stats = llm.engine.speculative_runner.stats
    native_tokens = [list(o.token_ids) for o in native]
    speculative_tokens = [list(o.token_ids) for o in speculative]
    assert native_tokens == speculative_tokens
    return dict(config={f: getattr(config, f) for f in (
                    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "total_ut_steps",
                    "initializer_range")},
                seed=seed, prompts=prompts, max_tokens=max_tokens, k=k, draft_loops=draft, target_loops=target,
                block=block, tokens=native_tokens,
                stats=dict(rounds=stats.rounds, drafted=stats.drafted_tokens, accepted=stats.accepted_tokens,
                           committed=stats.committed_tokens, verified_rows=stats.verified_rows))


def main():
    cases = {}
    g = torch.Generator().manual_seed(2024)
    tiny = OuroConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=128,
                      total_ut_steps=4, bos_token_id=0, eos_token_id=0)
    prompts = [torch.randint(1, 64, (n,), generator=g).tolist() for n in (1, 5, 2, 9)]
    cases["tiny_k3"] = run_case(tiny, 11, prompts, 24, 3, 2, 4, 256, 2)
    cases["tiny_k1_draft1"] = run_case(tiny, 12, prompts, 17, 1, 1, 4, 256, 2)
    config1 = OuroConfig(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-6,
                         rope_theta=10000.0, total_ut_steps=4, max_position_embeddings=256,
                         bos_token_id=0, eos_token_id=0)
    prompts = [torch.randint(1, 1024, (32,), generator=g).tolist() for _ in range(4)]
    cases["config1"] = run_case(config1, 7, prompts, 64, 4, 2, 4, 256, 16)
    torch.save(cases, HERE / "decode.pt")
    for name, case in cases.items():
        print(name, case["stats"], [len(t) for t in case["tokens"]])


if __name__ == "__main__":
    main()
