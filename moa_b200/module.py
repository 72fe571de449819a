"""Attention module and a Llama-architecture model around the MoA kernels.

``MoAAttention.forward`` keeps the contract of ``LlamaMixtureAttention.forward``
(MoA/models/llama/modeling_llama.py:206-332): MHA only, RoPE applied before caching (cached K carry
absolute positions), ``cache.update`` then attention (the new token is attended), ``sm_scale =
head_dim ** -0.5``, inference only, returns ``(attn_output, None, past_key_value)``.  What differs is
how many launches that takes: the three projections are one GEMM over a fused ``(3*H*D, hidden)`` weight
whose output the kernels read through strides (no split, no transpose copies), and in decode the rotary
embedding, the ring append, the attention and the bookkeeping are one kernel
(``StaticCircularCache.decode_attention``).

``MoALlamaModel`` / ``MoALlamaForCausalLM`` are the part of ``LlamaModel_MixtureAttention_forward`` (:52-203)
and ``LlamaModel_set_mixture_of_attention`` (:334-406) that belongs to this path: the
``StaticCircularCache`` is built from the plan on the first call with the reference's constants (sink 64,
minimum cache 128, split 64, ``moa_max_new_token``), the plan is installed, heads are optionally permuted
so equal capacities are adjacent, and — not in the reference, which is single-GPU — heads can be sharded
over the GPUs of a node (``shard_heads``).  Parameter names are those of a HuggingFace Llama checkpoint
(``model.layers.N.self_attn.q_proj.weight``, ``...mlp.gate_proj.weight``, ``lm_head.weight``), so such a
state dict loads as it is, and ``update_model_function`` turns a loaded HuggingFace Llama model into this
stack without copying its weights.  Nothing here calls into HuggingFace code; GEMMs, norms and the MLP are
plain torch ops (library kernels), the attention path is this package's kernels.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor, nn

from .attention import check_device_status, mixture_of_sparse_attention
from .cache import StaticCircularCache
from .plan import (
    moa_config_to_cache_config,
    moa_config_to_permutation,
    permute_attention_projection,
    permute_output_projection,
    prefill_block_visits,
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

    ``num_local_heads`` restricts the module to a shard of the heads (head sharding across GPUs): the q/k/v
    projections then produce only those heads and ``gather`` (a callable ``(B, q, H_local, D) ->
    (B, q, H, D)``, e.g. ``HeadSharding.all_gather``) rebuilds the full head dimension before
    ``o_proj``, which stays replicated.

    ``q_proj``, ``k_proj``, ``v_proj`` keep their checkpoint names, but their weights are three views of
    one ``(3*H_local*D, hidden)`` tensor, so that ``forward`` runs a single projection GEMM.  The views are
    rebuilt whenever one of the three weights has been replaced (loading, head permutation, sharding)."""

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
        self.gather: Optional[Callable[[Tensor], Tensor]] = None
        self.peer_gather = None     # a dist.PeerGather: decode steps then deliver their rows to every rank themselves
        self._qkv: Optional[Tensor] = None

    def fused_qkv_weight(self) -> Tensor:
        """The ``(3*H_local*D, hidden)`` weight of the single projection GEMM: rows of q, then k, then v
        (modeling_llama.py:234-236 as one matrix).  The three ``nn.Linear`` weights alias its thirds."""
        n = self.num_local_heads * self.head_dim
        w = self._qkv
        projs = (self.q_proj, self.k_proj, self.v_proj)
        if w is not None and all(p.weight.data_ptr() == w.data_ptr() + i * n * w.stride(0) * w.element_size()
                                 for i, p in enumerate(projs)):
            return w
        assert all(p.weight.shape == (n, self.hidden_size) for p in projs), "q/k/v projections must be (H_local*D, hidden)"
        w = torch.cat([p.weight.data for p in projs], dim=0)
        for i, p in enumerate(projs):
            p.weight = nn.Parameter(w[i * n:(i + 1) * n], requires_grad=False)
        self._qkv = w
        return w

    @torch.no_grad()
    def attend(self, hidden_states: Tensor, past_key_value: StaticCircularCache,
               position_embeddings: Tuple[Tensor, Tensor], out: Optional[Tensor] = None) -> Tensor:
        """Projection, rotary embedding, cache update and attention of this module's heads:
        ``(B, q, hidden) -> (B, q, H_local, D)`` (everything of ``forward`` before the gather and ``o_proj``).
        ``out`` (decode only) may be a ``(B, 1, H_local, D)`` slice of a gather buffer."""
        bsz, q_len, _ = hidden_states.shape
        H, D = self.num_local_heads, self.head_dim
        qkv = torch.nn.functional.linear(hidden_states, self.fused_qkv_weight()).view(bsz, q_len, 3, H, D)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))      # (B, H, q, D) views of the GEMM output
        cos, sin = position_embeddings
        sm_scale = D ** -0.5
        if q_len == 1:
            # one launch: rotary embedding of q and k, ring append, flash-decoding, bookkeeping
            if self.peer_gather is not None:    # ... and delivery of the rows to every rank: (B, 1, H, D) comes back
                return self.peer_gather.decode_and_gather(past_key_value, q, k, v, self.layer_idx, sm_scale,
                                                          rope=(cos, sin))
            return past_key_value.decode_attention(q, k, v, self.layer_idx, sm_scale, out=out, rope=(cos, sin))
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        past_key_value.update(k, v, self.layer_idx)
        return mixture_of_sparse_attention(
            q, k, v, sm_scale=sm_scale, attention_mask=None, attention_dropout=0.0,
            sink_size=past_key_value.static_cache_size[self.layer_idx],
            local_size=past_key_value.circular_cache_size[self.layer_idx],
            head_start_index=past_key_value.cache_head_start_index[self.layer_idx],
            head_valid_length=past_key_value.cache_valid_length[self.layer_idx])           # (B, q, H, D)

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
        if position_embeddings is None:
            assert position_ids is not None, "position_ids or position_embeddings are required"
            position_embeddings = rotary_cos_sin(position_ids, self.head_dim, self.rope_theta, hidden_states.dtype)
        attn = self.attend(hidden_states, past_key_value, position_embeddings)
        if self.gather is not None and attn.shape[2] != self.num_heads:
            attn = self.gather(attn)
        attn = attn.reshape(bsz, q_len, self.num_heads * self.head_dim)
        return self.o_proj(attn), None, past_key_value


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.float16, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        # one fused library kernel (fp32 statistics inside) instead of seven elementwise launches per norm
        return torch.nn.functional.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


class MoAMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, **kw)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, **kw)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, **kw)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class MoADecoderLayer(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, intermediate_size: int, layer_idx: int, rope_theta: float,
                 dtype, device, rms_norm_eps: float = 1e-6):
        super().__init__()
        self.self_attn = MoAAttention(hidden_size, num_heads, layer_idx, rope_theta, dtype, device)
        self.mlp = MoAMLP(hidden_size, intermediate_size, dtype, device)
        self.input_layernorm = RMSNorm(hidden_size, rms_norm_eps, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(hidden_size, rms_norm_eps, dtype=dtype, device=device)

    def forward(self, hidden_states, past_key_value, position_embeddings):
        h = self.input_layernorm(hidden_states)
        h, _, _ = self.self_attn(h, past_key_value=past_key_value, position_embeddings=position_embeddings)
        hidden_states = hidden_states + h
        return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))


class MoALlamaModel(nn.Module):
    """Llama-architecture decoder stack with MoA attention; parameter names as HuggingFace's ``LlamaModel``."""

    def __init__(self, num_layers: int, hidden_size: int, num_heads: int, intermediate_size: int,
                 vocab_size: int = 32000, rope_theta: float = 10000.0, dtype: torch.dtype = torch.float16,
                 device=None, rms_norm_eps: float = 1e-6):
        super().__init__()
        self.hidden_size, self.num_heads, self.rope_theta = hidden_size, num_heads, rope_theta
        self.embed_tokens = nn.Embedding(vocab_size, hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([
            MoADecoderLayer(hidden_size, num_heads, intermediate_size, i, rope_theta, dtype, device, rms_norm_eps)
            for i in range(num_layers)])
        self.norm = RMSNorm(hidden_size, rms_norm_eps, dtype=dtype, device=device)
        self.moa_config: Optional[Dict] = None
        self.local_moa_config: Optional[Dict] = None      # the plan of this rank's heads once heads are sharded
        self.head_shardings: Optional[List] = None
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
        assert self.head_shardings is None, "install the plan before sharding the heads"
        moa_config = copy.deepcopy(moa_config)
        self.moa_verbose, self.last_hidden_only, self.moa_max_new_token = moa_verbose, last_hidden_only, moa_max_new_token
        if permute_head:
            permutations, _ = moa_config_to_permutation(moa_config)
            for layer_id, layer in enumerate(self.layers):
                perm = permutations[layer_id]
                moa_config["alphas"][layer_id] = [moa_config["alphas"][layer_id][i] for i in perm]
                moa_config["betas"][layer_id] = [moa_config["betas"][layer_id][i] for i in perm]
                self._permute_heads(layer.self_attn, perm)
        self.use_moa = True
        self.moa_config = moa_config
        self.local_moa_config = None

    @staticmethod
    def _permute_heads(attn: MoAAttention, perm: Tensor) -> None:
        perm_dev = perm.to(attn.o_proj.weight.device)
        for proj in (attn.q_proj, attn.k_proj, attn.v_proj):
            permute_attention_projection(proj, perm_dev, attn.num_heads)
        permute_output_projection(attn.o_proj, perm_dev, attn.num_heads)

    def shard_heads(self, world_size: int, rank: int, seq_len: int, group=None, cost: str = "decode") -> None:
        """Keep only this rank's head shard of every layer (no counterpart in the single-GPU reference).

        Per layer the heads are placed on the ranks by longest-processing-time packing of their cost at
        context ``seq_len`` (``cost="decode"``: cache capacity, i.e. bytes per decode step;
        ``cost="prefill"``: visited 64x64 blocks); the q/k/v row blocks and the o_proj column blocks are
        permuted into shard order with the reference's ``permute_head`` mechanism, q/k/v are then cut down to
        the local rows, the caches built later hold the local heads only, and the attention outputs are
        all-gathered before the replicated ``o_proj``.  Call after ``set_mixture_of_attention`` and before the
        first forward; every rank must call it with the same plan."""
        from .dist import HeadSharding

        assert self.use_moa, "call set_mixture_of_attention(plan) first"
        assert self.head_shardings is None, "heads are already sharded"
        cfg = moa_config_to_cache_config(self.moa_config, seq_len=seq_len, max_new_token=self.moa_max_new_token,
                                         sink_size=64, minimum_cache_size=128, split_size=64, verbose=False)
        local = {"alphas": [], "betas": []}
        shardings = []
        D = self.hidden_size // self.num_heads
        for layer_id, layer in enumerate(self.layers):
            caps, static = cfg["cache_size"][layer_id], cfg["static_size"][layer_id]
            if cost == "prefill":
                costs = [prefill_block_visits(seq_len, [s // 64], [(c - s) // 64]) for c, s in zip(caps, static)]
            else:
                assert cost == "decode", "cost must be 'decode' or 'prefill'"
                costs = caps
            sh = HeadSharding(costs, world_size, rank, group=group)
            attn = layer.self_attn
            self._permute_heads(attn, torch.tensor(sh.order))
            rows = slice(rank * sh.heads_per_rank * D, (rank + 1) * sh.heads_per_rank * D)
            for proj in (attn.q_proj, attn.k_proj, attn.v_proj):
                proj.weight = nn.Parameter(proj.weight.data[rows].clone(), requires_grad=False)
                proj.out_features = sh.heads_per_rank * D
            attn.num_local_heads = sh.heads_per_rank
            attn._qkv = None
            attn.gather = sh.all_gather if world_size > 1 else None
            local["alphas"].append(sh.slice_plan(self.moa_config["alphas"][layer_id]))
            local["betas"].append(sh.slice_plan(self.moa_config["betas"][layer_id]))
            shardings.append(sh)
        self.head_shardings = shardings
        self.local_moa_config = local

    def enable_peer_gather(self, batch_size: int, wait_seconds: float = 2.0):
        """Decode steps of a head-sharded model deliver their output rows to every rank's gather buffer from
        inside the decode kernel (``dist.PeerGather``) instead of through an all-gather collective.  One set
        of buffers serves all layers.  Collective call (all ranks, after ``shard_heads``); returns the
        ``PeerGather`` (``check()`` reports a rank that went missing, ``close()`` releases the buffers)."""
        from .dist import PeerGather

        assert self.head_shardings is not None, "shard the heads first"
        pg = PeerGather(self.head_shardings[0], batch_size, self.hidden_size // self.num_heads, self.dtype,
                        self.device, wait_seconds)
        for layer in self.layers:
            layer.self_attn.peer_gather = pg
        return pg

    def new_cache(self, batch_size: int, seq_length: int) -> StaticCircularCache:
        """The cache the reference builds on the first forward (modeling_llama.py:93-112); with sharded heads,
        the cache of this rank's heads."""
        assert self.use_moa, "call set_mixture_of_attention(plan) first"
        plan = self.local_moa_config if self.local_moa_config is not None else self.moa_config
        cfg = moa_config_to_cache_config(plan, seq_len=seq_length, max_new_token=self.moa_max_new_token,
                                         sink_size=64, minimum_cache_size=128, split_size=64, verbose=self.moa_verbose)
        return StaticCircularCache(**cfg, batch_size=batch_size, head_dim=self.hidden_size // self.num_heads,
                                   device=self.device, dtype=self.dtype, update_cache_content=True)

    @torch.no_grad()
    def forward(self, input_ids: Optional[Tensor] = None, past_key_values: Optional[StaticCircularCache] = None,
                inputs_embeds: Optional[Tensor] = None, position_ids: Optional[Tensor] = None):
        """Returns ``(last_hidden_state, cache)``; ``last_hidden_state`` is ``(B, 1, hidden)`` when
        ``last_hidden_only`` (modeling_llama.py:195-199).  After a prefill (more than one token) the device
        status words are read once: a bounded wait that ran out inside the prefill kernel raises here instead
        of passing invalid activations on to the decode steps."""
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
        if seq_length > 1:
            check_device_status(inputs_embeds.device)
        hidden = self.norm(hidden)
        if self.last_hidden_only:
            hidden = hidden[:, -1:, :]
        return hidden, past_key_values


class MoALlamaForCausalLM(nn.Module):
    """``model`` (a ``MoALlamaModel``) + ``lm_head``, with the parameter names of HuggingFace's
    ``LlamaForCausalLM``: ``load_state_dict`` takes such a checkpoint's state dict as it is."""

    def __init__(self, num_layers: int, hidden_size: int, num_heads: int, intermediate_size: int,
                 vocab_size: int = 32000, rope_theta: float = 10000.0, dtype: torch.dtype = torch.float16,
                 device=None, rms_norm_eps: float = 1e-6):
        super().__init__()
        self.model = MoALlamaModel(num_layers, hidden_size, num_heads, intermediate_size, vocab_size, rope_theta,
                                   dtype, device, rms_norm_eps)
        self.lm_head = nn.Linear(hidden_size, vocab_size, bias=False, dtype=dtype, device=device)
        self.eval()

    @classmethod
    def from_config(cls, config, dtype: torch.dtype = torch.float16, device=None) -> "MoALlamaForCausalLM":
        """From the fields of a Llama ``config.json`` (a dict or an object with those attributes).  MHA only:
        ``num_key_value_heads`` must equal ``num_attention_heads`` (modeling_llama.py:220-224)."""
        get = (lambda k, d=None: config.get(k, d)) if isinstance(config, dict) else (lambda k, d=None: getattr(config, k, d))
        heads = get("num_attention_heads")
        kv = get("num_key_value_heads", heads) or heads
        assert kv == heads, "only support one key value group now (convert the checkpoint to MHA first)"
        theta = get("rope_theta")
        if theta is None:       # newer configs keep it inside rope_parameters
            params = get("rope_parameters") or {}
            theta = (params.get("rope_theta") if isinstance(params, dict) else getattr(params, "rope_theta", None)) or 10000.0
        return cls(get("num_hidden_layers"), get("hidden_size"), heads, get("intermediate_size"), get("vocab_size"),
                   float(theta), dtype, device, float(get("rms_norm_eps", 1e-6)))

    @classmethod
    def from_loaded(cls, hf_model) -> "MoALlamaForCausalLM":
        """Adopts a loaded HuggingFace-style Llama model (anything with ``.config`` and a Llama ``state_dict()``):
        same weights (shared, not copied, until a permutation or sharding replaces them), this package's
        attention path."""
        first = next(hf_model.parameters())
        with torch.device("meta"):
            new = cls.from_config(hf_model.config, dtype=first.dtype)
        state = {k: v for k, v in hf_model.state_dict().items() if not k.endswith("rotary_emb.inv_freq")}
        if "lm_head.weight" not in state:      # tied embeddings
            state["lm_head.weight"] = state["model.embed_tokens.weight"]
        new.load_state_dict(state, strict=True, assign=True)
        return new

    def set_mixture_of_attention(self, *args, **kwargs) -> None:
        self.model.set_mixture_of_attention(*args, **kwargs)

    @torch.no_grad()
    def forward(self, input_ids: Optional[Tensor] = None, past_key_values: Optional[StaticCircularCache] = None,
                inputs_embeds: Optional[Tensor] = None, position_ids: Optional[Tensor] = None):
        """Returns ``(logits, cache)``; logits of the last position only when ``model.last_hidden_only``."""
        hidden, cache = self.model(input_ids, past_key_values, inputs_embeds, position_ids)
        return self.lm_head(hidden), cache


class DecodeGraph:
    """One decode step of the whole model (every layer's projection GEMMs, fused decode launch, gather,
    ``o_proj``, MLP, and ``lm_head`` for a causal LM) captured once in a CUDA graph and replayed per token.

    Not in the reference, which launches every kernel of every layer from Python on each step; at decode batch
    sizes the GPU work of a layer is tens of microseconds and the launches dominate.  What has to live on the
    device for a replay to be exact does: the position (a device counter that the graph itself advances and the
    rotary tables are computed from), the ring write pointers and lengths (advanced by the decode kernel), and
    the call number of the cross-rank barrier.  The layer's token count is passed to the decode kernel by
    value, which is exact once every ring has left its static part — capture is refused before that.

    Use: run the prefill and one ordinary decode step (libraries initialise lazily on the first one), then::

        graph = DecodeGraph(model, cache)          # model: MoALlamaModel or MoALlamaForCausalLM
        out = graph.step(next_ids)                 # (B, 1, hidden) or (B, 1, vocab); overwritten by the next step

    With sharded heads every rank must capture and replay alike; a ``PeerGather`` needs an even number of
    layers (its two buffers alternate by call)."""

    def __init__(self, model, cache: StaticCircularCache):
        self.model = model
        self.cache = cache
        base = model.model if isinstance(model, MoALlamaForCausalLM) else model
        device, B = base.device, cache.batch_size
        for layer in range(cache.num_layers):
            if cache.get_seq_length(layer) <= max(cache._static_host[layer]):
                raise RuntimeError("DecodeGraph: capture once every ring has left its static part "
                                   "(the prompt plus the tokens decoded so far must exceed the sink size)")
        if any(l.self_attn.peer_gather is not None for l in base.layers) and len(base.layers) % 2:
            raise RuntimeError("DecodeGraph: the fused gather alternates two buffers by call and needs an even "
                               "number of layers per captured step")
        self.ids = torch.zeros(B, 1, dtype=torch.long, device=device)
        self.position = torch.full((1, 1), cache.get_seq_length(), dtype=torch.long, device=device)
        kv_len, cache_position = list(cache._kv_len), cache.cache_position
        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream(device))
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=stream):
            out, _ = model(self.ids, past_key_values=cache, position_ids=self.position)
            self.position.add_(1)
            self.out = out
        torch.cuda.current_stream(device).wait_stream(stream)
        # capturing ran the host side once without executing anything: take the host counters back
        cache._kv_len, cache.cache_position = kv_len, cache_position

    @torch.no_grad()
    def step(self, input_ids: Tensor) -> Tensor:
        self.ids.copy_(input_ids, non_blocking=True)
        self.graph.replay()
        self.cache._kv_len = [n + 1 for n in self.cache._kv_len]
        self.cache.cache_position += 1
        return self.out


class _ModelHolder:
    """``model.model`` indirection of HuggingFace causal-LM wrappers, for a bare ``MoALlamaModel``."""

    def __init__(self, model):
        self.model = model


def update_model_function(model, model_name: str):
    """Counterpart of MoA/models/interface.py:3-28: returns a model whose ``model.model`` has
    ``set_mixture_of_attention`` and runs this package's attention path.  Accepted: a
    ``MoALlamaForCausalLM`` (returned as it is), a bare ``MoALlamaModel`` (wrapped so that ``.model`` is it),
    or a loaded HuggingFace-style Llama causal LM (``.config``, ``.model.layers``, ``.lm_head``), which is
    converted with ``MoALlamaForCausalLM.from_loaded`` — the reference patches such a model's methods in
    place; here its weights move into a stack that does not depend on the installed transformers version."""
    name = model_name.lower()
    if not any(tag in name for tag in ("llama", "vicuna", "longchat")):
        raise NotImplementedError(f"Model {model_name} not implemented")
    if isinstance(model, MoALlamaForCausalLM):
        return model
    if isinstance(model, MoALlamaModel):
        return _ModelHolder(model)
    if hasattr(model, "config") and hasattr(model, "model") and hasattr(model.model, "layers") and hasattr(model, "lm_head"):
        return MoALlamaForCausalLM.from_loaded(model)
    assert hasattr(model, "model") and hasattr(model.model, "set_mixture_of_attention")
    return model
