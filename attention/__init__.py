"""The reference's import name for the operators this library rebuilds.

Callers of the reference write ``import attention`` and ``attention.gqa_decode(q, k_cache,
v_cache, block_table, context_lens)`` (attention/__init__.py:2-19,
benchmarks/bench_gqa_decode.py:43).  With this directory on ``sys.path`` in place of the
reference's package, the same lines run the B200 kernels of ``attention_b200``.  Only the
names of the rebuilt path exist here: the paged GQA decode front doors, ``kv_append``,
``gqa_prefill`` and the paged latent (MLA) decode operators.  ``sparse_mla`` is
``mla_decode`` with ``indices``, as in the reference (attention/sparse.py:23-24).  The
reference's Python oracle (``reference_gqa_decode``) is deliberately absent: checkers are
not part of the product.
"""

from attention_b200 import (gqa_decode, gqa_decode_auto, gqa_decode_split, gqa_prefill,
                            is_cuda_extension_loaded, kv_append, latent_kv_write, mla_decode,
                            mla_latent_attention, mla_query_absorb, mla_value_project,
                            validate_paged_metadata)
from attention_b200 import __version__


def sparse_mla(q_nope, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, indices, *,
               scale=None):
    """``mla_decode`` restricted to the logical tokens listed in ``indices`` ``[B,T,K]``."""
    return mla_decode(q_nope, q_rope, cache, block_table, lengths, positions, w_uk, w_uv,
                      scale=scale, indices=indices)


__all__ = [
    "gqa_decode", "gqa_decode_split", "gqa_decode_auto", "gqa_prefill", "kv_append",
    "is_cuda_extension_loaded", "latent_kv_write", "mla_query_absorb", "mla_value_project",
    "mla_latent_attention", "mla_decode", "sparse_mla", "validate_paged_metadata",
]
