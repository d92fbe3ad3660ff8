"""An Ouro-shaped looped language model around the B200 verify-step kernels.

This is the call-site side of the path (`vllm_rlt/models/ouro.py:171-291` of the reference):
embedding prelude, a stack of sandwich-norm decoder layers that is applied once per recurrent
loop with shared weights, final norm inside the recurrence, LM-head coda.  The GEMMs are
PyTorch (cuBLAS); everything between them is this package's kernels: fused RoPE + KV write,
paged attention, SiLU-and-Mul and the fused sandwich RMSNorm + residual (`fused=False` keeps
RMSNorm and RoPE as the reference's tensor expressions, for comparison).  Parameter names are
the reference's (checkpoint-compatible), so a reference `state_dict()` loads unchanged.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .activation import silu_and_mul, silu_and_mul_packed
from .attention import B200PagedAttention
from .kv_cache import kv_write
from .layers import rope_kv_write, sandwich_norm


@dataclass(frozen=True)
class LoopedLMConfig:
    """The architectural fields of the reference's OuroConfig (models/ouro.py:36-49)."""

    vocab_size: int = 49152
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    total_ut_steps: int = 4
    initializer_range: float = 0.02


def parameter_shapes(config: LoopedLMConfig) -> dict[str, tuple]:
    h, f = config.hidden_size, config.intermediate_size
    q, kv = config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim
    shapes = {"model.embed_tokens.weight": (config.vocab_size, h), "model.norm.weight": (h,),
              "model.early_exit_gate.weight": (1, h), "model.early_exit_gate.bias": (1,),
              "lm_head.weight": (config.vocab_size, h)}
    for layer in range(config.num_hidden_layers):
        p = f"model.layers.{layer}."
        shapes.update({
            p + "self_attn.q_proj.weight": (q, h), p + "self_attn.k_proj.weight": (kv, h),
            p + "self_attn.v_proj.weight": (kv, h), p + "self_attn.o_proj.weight": (h, q),
            p + "mlp.gate_proj.weight": (f, h), p + "mlp.up_proj.weight": (f, h),
            p + "mlp.down_proj.weight": (h, f),
            p + "input_layernorm.weight": (h,), p + "input_layernorm_2.weight": (h,),
            p + "post_attention_layernorm.weight": (h,), p + "post_attention_layernorm_2.weight": (h,),
        })
    return shapes


def seeded_parameter(name: str, shape, seed: int, std: float, device="cpu") -> torch.Tensor:
    """N(0, std) values for one named parameter from a generator seeded by (seed, name); norm
    weights are ones and biases zeros.  Order independent, so any subset can be rebuilt."""
    if name.endswith("norm.weight") or "layernorm" in name:
        return torch.ones(shape, device=device)
    if name.endswith(".bias"):
        return torch.zeros(shape, device=device)
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    generator = torch.Generator(device=device).manual_seed(int.from_bytes(digest[:7], "little"))
    return torch.randn(shape, generator=generator, device=device) * std


def seeded_state_dict(config: LoopedLMConfig, seed: int, device="cpu") -> dict[str, torch.Tensor]:
    """Random-init weights of the given shape (there is no checkpoint to load offline)."""
    return {name: seeded_parameter(name, shape, seed, config.initializer_range, device)
            for name, shape in parameter_shapes(config).items()}


def rms_norm(hidden: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """layers/normalization.py:20-23 of the reference: fp32 reduction, weight applied after the cast."""
    value = hidden.float()
    value = value * torch.rsqrt(value.square().mean(-1, keepdim=True) + eps)
    return weight * value.to(hidden.dtype)


def rotate_half(value: torch.Tensor) -> torch.Tensor:
    first, second = value.chunk(2, dim=-1)
    return torch.cat((-second, first), dim=-1)


class LoopedLM:
    """Inference-only looped LM: `prelude`, one `recurrent` loop over all layers, `coda`."""

    def __init__(self, config: LoopedLMConfig, state_dict: dict, device, dtype: torch.dtype,
                 attention: B200PagedAttention | None = None, fused: bool = True):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        missing = set(parameter_shapes(config)) - set(state_dict)
        if missing:
            raise ValueError(f"state dict lacks {sorted(missing)[:3]}...")
        self.w = {name: state_dict[name].to(device=self.device, dtype=dtype) for name in parameter_shapes(config)}
        self.attention = attention or B200PagedAttention()
        self.fused = fused
        # one projection for q, k and v: the rotary kernel reads its three column slices in place
        self.qkv = [torch.cat([self.w[f"model.layers.{layer}.self_attn.{n}_proj.weight"] for n in "qkv"])
                    for layer in range(config.num_hidden_layers)] if fused else None
        # and one for gate and up: SiLU-and-Mul reads the two column halves of its output in place
        self.gate_up = [torch.cat([self.w[f"model.layers.{layer}.mlp.{n}_proj.weight"] for n in ("gate", "up")])
                        for layer in range(config.num_hidden_layers)] if fused else None
        self.inv_freq = 1.0 / (config.rope_theta ** (
            torch.arange(0, config.head_dim, 2, dtype=torch.float32, device=self.device) / config.head_dim))

    def prelude(self, token_ids: torch.Tensor) -> torch.Tensor:
        return F.embedding(token_ids, self.w["model.embed_tokens.weight"])

    def rope(self, positions: torch.Tensor):
        """layers/rotary_embedding.py:54-64 of the reference (fp32 angles, cast to the model dtype)."""
        angles = positions.float().unsqueeze(-1) * self.inv_freq
        angles = torch.cat((angles, angles), dim=-1)
        return angles.cos().to(self.dtype).unsqueeze(1), angles.sin().to(self.dtype).unsqueeze(1)

    def recurrent(self, hidden, positions, key_pool, value_pool, write_blocks, write_offsets, block_tables,
                  context_lengths, packed=None, write_mask=None):
        """One recurrent loop: every layer writes its K/V rows, attends, and runs the MLP.

        key_pool / value_pool: `[blocks, layers, block_size, kv_heads, head_dim]`; the addressing
        tensors select the depth plane (they are the same for all layers of the loop, so the
        attention work list is planned once).  Returns the normalised hidden state, which is the
        next loop's input and the coda's input (models/ouro.py:283-291).

        `packed = (cu_seqlens_q, max_seqlen_q)` switches to the packed form for prompts: one
        block-table row and one context length per sequence, rows of a sequence consecutive
        (`AttentionBackend.prefill`).  `write_mask` (bool [rows]) keeps inactive rows from writing K/V
        (their context length should be 0 so that they attend to nothing)."""
        if self.fused:
            return self._recurrent_fused(hidden, positions, key_pool, value_pool, write_blocks, write_offsets,
                                         block_tables, context_lengths, packed=packed, write_mask=write_mask)
        c, w = self.config, self.w
        cos, sin = self.rope(positions)
        rows = hidden.shape[0]
        with self.attention.shared_plan():
            for layer in range(c.num_hidden_layers):
                p = f"model.layers.{layer}."
                x = rms_norm(hidden, w[p + "input_layernorm.weight"], c.rms_norm_eps)
                q = F.linear(x, w[p + "self_attn.q_proj.weight"]).view(rows, -1, c.head_dim)
                k = F.linear(x, w[p + "self_attn.k_proj.weight"]).view(rows, -1, c.head_dim)
                v = F.linear(x, w[p + "self_attn.v_proj.weight"]).view(rows, -1, c.head_dim)
                q = q * cos + rotate_half(q) * sin
                k = k * cos + rotate_half(k) * sin
                kc, vc = key_pool[:, layer], value_pool[:, layer]
                kv_write(kc, vc, k, v, write_blocks, write_offsets, write_mask=write_mask)
                attended = self._attend(q.contiguous(), kc, vc, block_tables, context_lengths, packed)
                attended = F.linear(attended.reshape(rows, -1), w[p + "self_attn.o_proj.weight"])
                hidden = hidden + rms_norm(attended, w[p + "input_layernorm_2.weight"], c.rms_norm_eps)
                x = rms_norm(hidden, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
                gate = F.linear(x, w[p + "mlp.gate_proj.weight"])
                up = F.linear(x, w[p + "mlp.up_proj.weight"])
                mlp = F.linear(silu_and_mul(gate, up), w[p + "mlp.down_proj.weight"])
                hidden = hidden + rms_norm(mlp, w[p + "post_attention_layernorm_2.weight"], c.rms_norm_eps)
        return rms_norm(hidden, w["model.norm.weight"], c.rms_norm_eps)

    def _attend(self, q, key_cache, value_cache, block_tables, context_lengths, packed):
        if packed is None:
            return self.attention(q, key_cache, value_cache, block_tables, context_lengths)
        return self.attention.prefill(q, key_cache, value_cache, block_tables, context_lengths, *packed)

    def _recurrent_fused(self, hidden, positions, key_pool, value_pool, write_blocks, write_offsets, block_tables,
                         context_lengths, active_rows=None, packed=None, write_mask=None):
        """The same loop with nine launches per layer (ten when the attention merges chunks): QKV GEMM,
        rope_kv_write, attention, O GEMM, sandwich_norm (residual add + the MLP's input norm), one gate-and-up
        GEMM, silu_and_mul_packed, down GEMM, sandwich_norm (residual add + the next layer's input norm, or the
        final norm).
        `active_rows` (0-dim int32) marks padding rows of a captured graph: they write no K/V."""
        c, w = self.config, self.w
        cos, sin = self.rope(positions)
        rows = hidden.shape[0]
        q_width, kv_width = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        stream = None                                                  # residual stream, owned by this call
        x, _ = sandwich_norm(hidden, w["model.layers.0.input_layernorm.weight"], c.rms_norm_eps)
        with self.attention.shared_plan():
            for layer in range(c.num_hidden_layers):
                p = f"model.layers.{layer}."
                qkv = F.linear(x, self.qkv[layer])
                q = qkv[:, :q_width].view(rows, -1, c.head_dim)
                k = qkv[:, q_width:q_width + kv_width].view(rows, -1, c.head_dim)
                v = qkv[:, q_width + kv_width:].view(rows, -1, c.head_dim)
                kc, vc = key_pool[:, layer], value_pool[:, layer]
                q = rope_kv_write(q, k, v, cos, sin, kc, vc, write_blocks, write_offsets, write_mask=write_mask,
                                  active_rows=active_rows)
                attended = self._attend(q, kc, vc, block_tables, context_lengths, packed)
                attended = F.linear(attended.view(rows, -1), w[p + "self_attn.o_proj.weight"])
                stream, x = sandwich_norm(attended, w[p + "input_layernorm_2.weight"], c.rms_norm_eps,
                                          hidden if stream is None else stream,
                                          w[p + "post_attention_layernorm.weight"], in_place=stream is not None)
                mlp = F.linear(silu_and_mul_packed(F.linear(x, self.gate_up[layer])), w[p + "mlp.down_proj.weight"])
                following = (w[f"model.layers.{layer + 1}.input_layernorm.weight"]
                             if layer + 1 < c.num_hidden_layers else w["model.norm.weight"])
                stream, x = sandwich_norm(mlp, w[p + "post_attention_layernorm_2.weight"], c.rms_norm_eps, stream,
                                          following, in_place=True)
        return x

    def coda(self, hidden: torch.Tensor) -> torch.Tensor:
        return F.linear(hidden, self.w["lm_head.weight"])
