"""Attention module and a small Llama-architecture model around the MoA kernels.

``MoAAttention.forward`` keeps the contract of ``LlamaMixtureAttention.forward``
(MoA/models/llama/modeling_llama.py:206-332): MHA only, RoPE applied before caching (cached K carry
absolute positions), ``cache.update`` then attention (the new token is attended), ``sm_scale =
head_dim ** -0.5``, inference only, returns ``(attn_output, None, past_key_value)``.  In decode the
append and the attention are one kernel launch (``StaticCircularCache.decode_attention``).

``MoALlamaModel`` is the part of ``LlamaModel_MixtureAttention_forward`` (:52-203) and
``LlamaModel_set_mixture_of_attention`` (:334-406) that belongs to this path: it builds the
``StaticCircularCache`` from the plan on the first call with the reference's constants
(sink 64, minimum cache 128, split 64, ``moa_max_new_token``), installs the plan, and optionally
permutes heads so equal capacities are adjacent.  It does not depend on HuggingFace internals; GEMMs,
norms and the MLP are plain torch ops (library kernels), the attention path is this package's kernels.
"""
from __future__ import annotations

import copy
import math
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor, nn

from .attention import mixture_of_sparse_attention
from .cache import StaticCircularCache
from .plan import (
    moa_config_to_cache_config,
    moa_config_to_permutation,
    permute_attention_projection,
    permute_output_projection,
)


def rotary_cos_sin(position_ids: Tensor, head_dim: int, theta: float, dtype: torch.dtype) -> Tuple[Tensor, Tensor]:
    """(B, q, D) cos/sin tables, computed in fp32 and cast to the model dtype as the Llama rotary
    embedding does (shared by all layers of a forward, modeling_llama.py:137)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=position_ids.device) / head_dim))
    freqs = position_ids[:, :, None].float() * inv_freq[None, None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rotary_pos_emb(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> Tuple[Tensor, Tensor]:
    """Rotary embedding of q and k, in place, in one kernel pass (``moa_rope_qk``).  q, k ``(B, H, q_len, D)``
    with the same strides and a contiguous last dim; cos, sin ``(B, q_len, D)`` (or ``(1, q_len, D)``) in their
    dtype.  Returns ``(q, k)`` (the same tensors)."""
    from . import _lib

    B, H, N, D = q.shape
    assert k.shape == q.shape and q.stride() == k.stride() and q.stride(-1) == 1
    assert cos.shape[-2:] == (N, D) and cos.stride() == sin.stride() and cos.stride(-1) == 1 and cos.dtype == q.dtype
    assert cos.shape[0] in (1, B)
    cs_b = 0 if cos.shape[0] == 1 else cos.stride(0)
    with torch.cuda.device(q.device):
        _lib.check("moa_rope_qk", _lib.lib.moa_rope_qk(
            q.data_ptr(), k.data_ptr(), q.stride(0), q.stride(1), q.stride(2), cos.data_ptr(), sin.data_ptr(),
            cs_b, cos.stride(1), B, H, N, D, _lib.dtype_code(q.dtype), _lib.current_stream(q.device)))
    return q, k


class MoAAttention(nn.Module):
    """Multi-head attention with per-head sink + sliding-window spans.

    ``head_ids`` restricts the module to a shard of the heads (head sharding across GPUs): the q/k/v
    projections then produce only those heads and ``gather`` (a callable ``(B, q, H_local, D) ->
    (B, q, H, D)``, e.g. ``HeadSharding.all_gather``) rebuilds the full head dimension before
    ``o_proj``, which stays replicated."""

    def __init__(self, hidden_size: int, num_heads: int, layer_idx: int, rope_theta: float = 10000.0,
                 dtype: torch.dtype = torch.float16, device=None, num_local_heads: Optional[int] = None):
        super().__init__()
        assert hidden_size % num_heads == 0
        self.hidden_size, self.num_heads, self.layer_idx = hidden_size, num_heads, layer_idx
        self.head_dim = hidden_size // num_heads
        self.num_key_value_groups = 1      # MHA only, as the reference (modeling_llama.py:220-224)
        self.num_local_heads = num_local_heads if num_local_heads is not None else num_heads
        self.rope_theta = rope_theta
        kw = dict(bias=False, dtype=dtype, device=device)
        self.q_proj = nn.Linear(hidden_size, self.num_local_heads * self.head_dim, **kw)
        self.k_proj = nn.Linear(hidden_size, self.num_local_heads * self.head_dim, **kw)
        self.v_proj = nn.Linear(hidden_size, self.num_local_heads * self.head_dim, **kw)
        self.o_proj = nn.Linear(num_heads * self.head_dim, hidden_size, **kw)
        self.gather = None

    @torch.no_grad()
    def forward(self, hidden_states: Tensor, attention_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None, past_key_value: Optional[StaticCircularCache] = None,
                output_attentions: bool = False, use_cache: bool = False, cache_position: Optional[Tensor] = None,
                position_embeddings: Optional[Tuple[Tensor, Tensor]] = None, **kwargs):
        assert self.num_key_value_groups == 1, "only support one key value group now"
        if output_attentions:
            raise NotImplementedError("output_attentions is not supported in mixture of attention")
        assert not self.training, "only support inference now"
        assert isinstance(past_key_value, StaticCircularCache), "MoAAttention needs a StaticCircularCache"
        bsz, q_len, _ = hidden_states.shape
        H, D = self.num_local_heads, self.head_dim
        q = self.q_proj(hidden_states).view(bsz, q_len, H, D).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, H, D).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, H, D).transpose(1, 2)
        if position_embeddings is None:
            assert position_ids is not None, "position_ids or position_embeddings are required"
            position_embeddings = rotary_cos_sin(position_ids, D, self.rope_theta, hidden_states.dtype)
        cos, sin = position_embeddings
        sm_scale = D ** -0.5
        if q_len == 1:
            # one launch: rotary embedding of q and k, ring append, flash-decoding, bookkeeping
            attn = past_key_value.decode_attention(q, k, v, self.layer_idx, sm_scale, rope=(cos, sin))   # (B, 1, H, D)
        else:
            q, k = apply_rotary_pos_emb(q, k, cos, sin)
            past_key_value.update(k, v, self.layer_idx)
            attn = mixture_of_sparse_attention(
                q, k, v, sm_scale=sm_scale, attention_mask=None, attention_dropout=0.0,
                sink_size=past_key_value.static_cache_size[self.layer_idx],
                local_size=past_key_value.circular_cache_size[self.layer_idx],
                head_start_index=past_key_value.cache_head_start_index[self.layer_idx],
                head_valid_length=past_key_value.cache_valid_length[self.layer_idx])           # (B, q, H, D)
        if self.gather is not None:
            attn = self.gather(attn)
        attn = attn.reshape(bsz, q_len, self.num_heads * D)
        return self.o_proj(attn), None, past_key_value


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.float16, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class MoADecoderLayer(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, intermediate_size: int, layer_idx: int, rope_theta: float,
                 dtype, device, num_local_heads: Optional[int] = None):
        super().__init__()
        self.self_attn = MoAAttention(hidden_size, num_heads, layer_idx, rope_theta, dtype, device, num_local_heads)
        kw = dict(bias=False, dtype=dtype, device=device)
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, **kw)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, **kw)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, **kw)
        self.input_layernorm = RMSNorm(hidden_size, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(hidden_size, dtype=dtype, device=device)

    def forward(self, hidden_states, past_key_value, position_embeddings):
        h = self.input_layernorm(hidden_states)
        h, _, _ = self.self_attn(h, past_key_value=past_key_value, position_embeddings=position_embeddings)
        hidden_states = hidden_states + h
        h = self.post_attention_layernorm(hidden_states)
        h = self.down_proj(torch.nn.functional.silu(self.gate_proj(h)) * self.up_proj(h))
        return hidden_states + h


class MoALlamaModel(nn.Module):
    """Llama-architecture decoder stack with MoA attention (random-init unless weights are loaded)."""

    def __init__(self, num_layers: int, hidden_size: int, num_heads: int, intermediate_size: int,
                 vocab_size: int = 32000, rope_theta: float = 10000.0, dtype: torch.dtype = torch.float16,
                 device=None):
        super().__init__()
        self.hidden_size, self.num_heads, self.rope_theta = hidden_size, num_heads, rope_theta
        self.embed_tokens = nn.Embedding(vocab_size, hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([
            MoADecoderLayer(hidden_size, num_heads, intermediate_size, i, rope_theta, dtype, device)
            for i in range(num_layers)])
        self.norm = RMSNorm(hidden_size, dtype=dtype, device=device)
        self.moa_config: Optional[Dict] = None
        self.use_moa = False
        self.moa_verbose = False
        self.last_hidden_only = True
        self.moa_max_new_token = 1024
        self.eval()

    @property
    def dtype(self):
        return self.embed_tokens.weight.dtype

    @property
    def device(self):
        return self.embed_tokens.weight.device

    def set_mixture_of_attention(self, moa_config: Dict, permute_head: bool = False, moa_verbose: bool = False,
                                 moa_max_new_token: int = 1024, last_hidden_only: bool = True,
                                 sparse_prefill: bool = True) -> None:
        """Install a plan ``{"alphas": [[...]], "betas": [[...]]}``  (modeling_llama.py:334-406).
        ``permute_head`` sorts every layer's heads by (alpha, beta) and permutes the q/k/v row blocks
        and the o_proj column blocks accordingly, so the model computes the same function."""
        assert sparse_prefill, "only support sparse prefill now"
        assert len(moa_config["alphas"]) == len(self.layers) == len(moa_config["betas"])
        moa_config = copy.deepcopy(moa_config)
        self.moa_verbose, self.last_hidden_only, self.moa_max_new_token = moa_verbose, last_hidden_only, moa_max_new_token
        if permute_head:
            permutations, _ = moa_config_to_permutation(moa_config)
            for layer_id, layer in enumerate(self.layers):
                perm = permutations[layer_id]
                moa_config["alphas"][layer_id] = [moa_config["alphas"][layer_id][i] for i in perm]
                moa_config["betas"][layer_id] = [moa_config["betas"][layer_id][i] for i in perm]
                attn = layer.self_attn
                perm_dev = perm.to(attn.q_proj.weight.device)
                permute_attention_projection(attn.q_proj, perm_dev, attn.num_heads)
                permute_attention_projection(attn.k_proj, perm_dev, attn.num_heads)
                permute_attention_projection(attn.v_proj, perm_dev, attn.num_heads)
                permute_output_projection(attn.o_proj, perm_dev, attn.num_heads)
        self.use_moa = True
        self.moa_config = moa_config

    def new_cache(self, batch_size: int, seq_length: int) -> StaticCircularCache:
        """The cache the reference builds on the first forward (modeling_llama.py:93-112)."""
        assert self.use_moa, "call set_mixture_of_attention(plan) first"
        cfg = moa_config_to_cache_config(self.moa_config, seq_len=seq_length, max_new_token=self.moa_max_new_token,
                                         sink_size=64, minimum_cache_size=128, split_size=64, verbose=self.moa_verbose)
        return StaticCircularCache(**cfg, batch_size=batch_size, head_dim=self.hidden_size // self.num_heads,
                                   device=self.device, dtype=self.dtype, update_cache_content=True)

    @torch.no_grad()
    def forward(self, input_ids: Optional[Tensor] = None, past_key_values: Optional[StaticCircularCache] = None,
                inputs_embeds: Optional[Tensor] = None, position_ids: Optional[Tensor] = None):
        """Returns ``(last_hidden_state, cache)``; ``last_hidden_state`` is ``(B, 1, hidden)`` when
        ``last_hidden_only`` (modeling_llama.py:195-199)."""
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("specify exactly one of input_ids and inputs_embeds")
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        batch_size, seq_length = inputs_embeds.shape[:2]
        if not isinstance(past_key_values, StaticCircularCache):
            past_key_values = self.new_cache(batch_size, seq_length)
        if position_ids is None:
            past = past_key_values.get_seq_length()
            position_ids = torch.arange(past, past + seq_length, device=inputs_embeds.device).unsqueeze(0)
        head_dim = self.hidden_size // self.num_heads
        pos_emb = rotary_cos_sin(position_ids.expand(batch_size, -1) if position_ids.shape[0] == 1 else position_ids,
                                 head_dim, self.rope_theta, inputs_embeds.dtype)
        hidden = inputs_embeds
        for layer in self.layers:
            hidden = layer(hidden, past_key_values, pos_emb)
        hidden = self.norm(hidden)
        if self.last_hidden_only:
            hidden = hidden[:, -1:, :]
        return hidden, past_key_values


class _ModelHolder:
    """``model.model`` indirection of HuggingFace causal-LM wrappers."""

    def __init__(self, model):
        self.model = model


def update_model_function(model, model_name: str):
    """Counterpart of MoA/models/interface.py:3-28: for llama/vicuna/longchat style names the model must
    expose ``model.model.set_mixture_of_attention``; a ``MoALlamaModel`` already does, a bare one is wrapped."""
    name = model_name.lower()
    if not any(tag in name for tag in ("llama", "vicuna", "longchat")):
        raise NotImplementedError(f"model name {model_name!r} is not a Llama-architecture model")
    if isinstance(model, MoALlamaModel):
        return _ModelHolder(model)
    assert hasattr(model, "model") and hasattr(model.model, "set_mixture_of_attention")
    return model
