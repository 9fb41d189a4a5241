"""B200-native paged grouped-query decode attention (drop-in for the reference's
``attention.gqa_decode`` path) and the operators either side of it."""

from .core import (gqa_decode, gqa_decode_auto, gqa_decode_split, gqa_prefill,
                   is_cuda_extension_loaded, kv_append, workspace_bytes)
from .mla import (latent_kv_write, mla_decode, mla_latent_attention, mla_query_absorb,
                  mla_value_project)
from .validation import validate_paged_metadata

__all__ = [
    "gqa_decode", "gqa_decode_split", "gqa_decode_auto", "gqa_prefill", "kv_append",
    "is_cuda_extension_loaded", "validate_paged_metadata", "workspace_bytes",
    "mla_decode", "mla_latent_attention", "mla_query_absorb", "mla_value_project", "latent_kv_write",
]
__version__ = "0.1.0"
