"""B200-native drop-in for the attention operators of flash-sparse-attention.

Same import paths and signatures as the reference package (``flash_sparse_attn/__init__.py:5-18``);
the compute runs in hand-written sm_100a CUDA kernels loaded from ``libfsa_b200.so``.
"""

__version__ = "2.0.6+b200"

from flash_sparse_attn.ops.triton.interface import (  # noqa: F401
    flash_dense_attn_func,
    flash_dense_attn_varlen_func,
    flash_dense_attn_varlen_with_kvcache_func,
    flash_dense_attn_with_kvcache_func,
    flash_gated_attn_func,
    flash_gated_attn_varlen_func,
    flash_gated_attn_varlen_with_kvcache_func,
    flash_gated_attn_with_kvcache_func,
    flash_sparse_attn_func,
    flash_sparse_attn_varlen_func,
    flash_sparse_attn_varlen_with_kvcache_func,
    flash_sparse_attn_with_kvcache_func,
)
from flash_sparse_attn._lib import check_status  # noqa: F401
from flash_sparse_attn.ops.triton.utils import deterministic_enabled, set_deterministic  # noqa: F401
