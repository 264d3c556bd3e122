"""b200attn: B200 (sm_100a) attention + paged KV-cache backend.

Host-side mirror of the attention path of tt-xla's vLLM plugin
(integrations/vllm_plugin/vllm_tt/attention_impls/attention.py) over a C-ABI library of
hand-written CUDA kernels.  There is no CPU path: every op raises when the CUDA library or a
CUDA device is missing.
"""
from . import _lib, ops  # noqa: F401
from .backend import (  # noqa: F401
    B200Attention,
    B200AttentionBackend,
    B200AttentionBackendImpl,
    B200AttentionMetadataBuilder,
    B200Metadata,
)

__all__ = [
    "ops",
    "B200Attention",
    "B200AttentionBackend",
    "B200AttentionBackendImpl",
    "B200AttentionMetadataBuilder",
    "B200Metadata",
]
