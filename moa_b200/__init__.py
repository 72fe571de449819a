"""moa_b200 — B200-native kernels behind MoA's attention API.

Drop-in names (same signatures as thu-nics/MoA):
``mixture_of_sparse_attention`` (MoA/kernels/mixture_of_attention.py:358),
``StaticCircularCache`` and ``moa_config_to_cache_config`` (MoA/attention/cache_utils.py:644, 1183),
``moa_config_to_permutation`` (MoA/attention/permutation_utils.py:219).

Importing the package loads ``libmoa_b200.so``; it raises if the library has not been built.
"""
from ._lib import LIB_PATH, MoaError  # noqa: F401  (loads the library, fails loudly if absent)
from .attention import check_device_status, mixture_of_sparse_attention, sparse_decode, sparse_prefill  # noqa: F401
from .cache import StaticCircularCache  # noqa: F401
from .dist import HeadSharding, PeerGather  # noqa: F401
from .module import DecodeGraph, MoAAttention, MoALlamaForCausalLM, MoALlamaModel, update_model_function  # noqa: F401
from .plan import (  # noqa: F401
    decode_bytes,
    load_plan,
    moa_config_to_cache_config,
    moa_config_to_permutation,
    permute_attention_projection,
    permute_output_projection,
    prefill_block_visits,
    prefill_flops,
    shard_heads,
)

__all__ = [
    "mixture_of_sparse_attention", "sparse_prefill", "sparse_decode", "check_device_status",
    "StaticCircularCache", "moa_config_to_cache_config", "moa_config_to_permutation",
    "permute_attention_projection", "permute_output_projection", "load_plan",
    "prefill_block_visits", "prefill_flops", "decode_bytes", "shard_heads", "MoaError", "LIB_PATH",
    "MoAAttention", "MoALlamaModel", "MoALlamaForCausalLM", "update_model_function", "HeadSharding", "PeerGather", "DecodeGraph",
]
