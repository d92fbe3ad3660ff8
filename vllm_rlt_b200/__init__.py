"""B200-native (sm_100a) self-speculative verify step for looped language models.

Hand-written CUDA kernels behind a C ABI (``include/rlt_verify.h``,
``vllm_rlt_b200/librlt_verify.so``) plus the thin PyTorch host layer that mirrors the
attention-backend, sampler, speculative and ``torch.ops.vllm_rlt`` interfaces of vllm-rlt
for this one path.  There is no CPU or library fallback: importing is cheap, the first call
raises if the CUDA library has not been built.
"""

from ._capi import NativeLibraryMissing, load as load_library
from .activation import register_torch_op, silu_and_mul, silu_and_mul_packed
from .attention import (B200_CAPABILITIES, AttentionBackend, B200PagedAttention, BackendCapabilities,
                        create_backend)
from .decoder import DecodeStats, GraphedLoops, PagedKV, SelfSpeculativeDecoder
from .prefix_cache import PrefixIndex
from .kv_cache import RollbackResult, finalize_tokens, kv_write, rollback
from .layers import rope_kv_write, sandwich_norm
from .looped_lm import LoopedLM, LoopedLMConfig, seeded_state_dict
from .runner import (B200SpeculativeRunner, KVCacheManagerView, ModelRunnerOutput, Request, SamplingParams, ScheduledRequest,
                     SchedulerOutput, SpeculativeConfig, SpeculativeRoundTicket, SpeculativeStats)
from .speculative import (PipelineState, SpeculativeResult, accept_greedy, accept_rejection, argmax_rows,
                          decode_result, pipeline_shift, probabilities, raise_for_status, round_uniforms,
                          sample_rows)

__all__ = [
    "AttentionBackend", "B200PagedAttention", "DecodeStats", "GraphedLoops", "LoopedLM", "LoopedLMConfig", "PagedKV", "PrefixIndex",
    "SelfSpeculativeDecoder", "seeded_state_dict", "B200_CAPABILITIES", "BackendCapabilities",
    "NativeLibraryMissing", "RollbackResult", "SpeculativeResult", "accept_greedy", "accept_rejection",
    "argmax_rows", "PipelineState", "create_backend", "decode_result", "finalize_tokens", "pipeline_shift", "kv_write", "load_library", "probabilities", "raise_for_status",
    "register_torch_op", "rollback", "rope_kv_write", "sample_rows", "sandwich_norm", "silu_and_mul",
    "B200SpeculativeRunner", "ModelRunnerOutput", "Request", "SamplingParams", "ScheduledRequest", "SchedulerOutput",
    "SpeculativeConfig", "SpeculativeRoundTicket", "SpeculativeStats", "round_uniforms", "silu_and_mul_packed",
    "KVCacheManagerView",
]
