"""Ragged-batch model for hybrid layer stacks: every layer names its own token mixer — attention over the paged cache
(per-head keys and values, or one latent vector per token), a gated-delta-rule (one decay per head, or per head and
key channel), state-space-duality or matrix-memory LSTM recurrence — and may or may not have a feed-forward (gated,
biased, or a mixture of experts); a span of layers can be executed several times in a row with the same weights, and
single layers can borrow another layer's weights, every execution with its own cache or state.

The stack is data (:class:`HybridSpec`), as :class:`~.inference_transformer_base.ArchSpec` is for the uniform
transformer family; per-architecture policies (``fomalix/policy.py``) fill it from a checkpoint's configuration and fuse
the checkpoint's tensors into the projection layouts the mixer modules declare.

Three layer forms (``HybridSpec.block_form``).  ``"sandwich"``: ``x += post_norm(sublayer(pre_norm(x)))``.
``"pre_scaled"``: ``x += m * sublayer(pre_norm(x))`` with one multiplier ``m`` for the whole stack (with ``layer_scale``
also a learned scale per layer, sublayer and channel: ``x += m * ls (.) sublayer(pre_norm(x))``; with
``norm_weight_offset`` the norms multiply by ``offset + w``), and optionally a
per-layer token input behind the feed-forward: ``x += m * rms_norm(proj(gelu(gate x) * e))`` where ``e`` is the layer's
part of one more embedding row of the token (``token_side_dim`` channels per layer).
``"post_scaled"``: ``x += scale (.) post_norm(sublayer(x + conv(x)))`` -- no pre-norm, a post-norm with one gain, a
per-channel scale, a short causal filter with a skip path in front of every sublayer (its last inputs are state of the
sequence), and optionally the stream handed to the next layer is a learned mixture of the embedding and of all
layers' results so far (``depth_mix``).

Numerics: the residual stream, norms, softmax, recurrences and their gates are fp32; projections, short convolutions'
inputs, the KV cache and the sublayer outputs use ``spec.dtype`` (bf16 when serving; fp32 evaluates everything in
32-bit, matrix products included).  Per layer execution: ``x += post_norm(mixer(pre_norm(x)))`` then, if the layer has a
feed-forward, ``x += post_norm(ff(pre_norm(x)))``; closing one sublayer and opening the next is one kernel
(``fp32_sandwich_rms``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ....ops import functional as F
from ..config_v2 import RaggedInferenceEngineConfig
from ..inference_utils import ActivationType, DtypeEnum, NormTypeEnum, ceil_div
from ..kernels import mixer_ops as M
from ..modules import heuristics
from ..modules.configs import (DSEmbeddingsConfig, DSLinearConfig, DSMoEConfig, DSNormConfig, DSRecurrentMixerConfig,
                               DSSelfAttentionConfig, DistanceBiasConfig, MaskingType, PositionalEmbeddingType,
                               RotaryScalingConfig, RotateHalfConfig)
from ..ragged.kv_cache import KVCacheConfig
from ..ragged.state_pool import StatePoolConfig
from .inference_transformer_base import DSInferenceModelBase, LayerWeights


@dataclass
class HybridLayerSpec:
    kind: str                      # "attention" | "latent_attention" | "delta" | "channel_delta" | "ssd" | "mlstm"
    n_heads: int
    n_heads_kv: int                             # key/value heads (attention), key/query heads (delta), groups (ssd)
    key_dim: int                                # query/key head size, or state size per group (ssd)
    value_dim: int
    attn_scale: float = 1.0
    chunk_size: int = 0                         # attention: 0 = plain causal, else chunk-local
    qk_unit_rms: bool = False
    sink: bool = False
    qkv_bias: bool = False
    conv_taps: int = 1
    norm_groups: int = 1
    ff_dim: int = 0                             # 0: the layer has no feed-forward
    ff_activation: str = "gelu"
    ff_kind: str = "gated"                      # "gated": down(act(gate) * up); "biased": down(act(up + b)) + b; "moe"
    n_experts: int = 0                          # moe: experts are gated feed-forwards of ff_dim channels
    top_k: int = 1
    moe_score: str = "softmax"
    moe_weight_input: bool = False
    moe_renormalize: bool = False               # the chosen experts' scores are divided by their sum
    window: int = 0                             # attention: > 0 = the query and the window - 1 positions before it
    q_rank: int = 0                             # latent attention: query latent, key/value latent, rotated channels
    kv_rank: int = 0
    rot_dim: int = 0
    rot_dims: int = 0                           # how many of the rot_dim channels turn (in interleaved pairs)
    rot_base: float = 10000.0
    gate_cap: float = 0.0                       # mlstm
    # attention with filtered projections (``conv_taps`` taps on q | k | v), a weighted q/k norm, a query temperature,
    # a learned distance-bucket bias (``dist_rows`` table rows, last row from distance ``dist_far`` on) and a gate
    qk_norm_weight: bool = False
    q_temp_coef: float = 0.0
    q_temp_every: int = 1
    dist_rows: int = 0
    dist_far: int = 0
    out_gate: bool = False
    ff_gated: bool = True                       # moe: experts are down(act(gate) * up); False: down(act(up))
    router_bias: bool = False
    shared_ff_dim: int = 0                      # moe: a shared expert of this width, gated by a sigmoid per token
    # latent attention: queries straight from the input (no query latent), one gate per head instead of one per output
    # channel (``out_gate``), wavelength-dependent slowing of the rotation (factor, original context, fast, slow turns)
    q_direct: bool = False
    gate_per_head: bool = False
    rot_scaling: Optional[Tuple[float, float, float, float]] = None
    # moe: group-limited choice by score + correction, weights rescaled, identity experts behind the real ones, clamp of
    # the experts' gated activation
    moe_correction: bool = False
    moe_groups: int = 1
    moe_keep_groups: int = 1
    moe_scale: float = 1.0
    moe_identity: int = 0
    ff_limit: float = 0.0


@dataclass
class HybridSpec:
    vocab_size: int
    model_dim: int
    layers: List[HybridLayerSpec]
    norm_eps: float = 1e-5
    embed_scale: float = 1.0
    sinusoid_base: Optional[float] = 10000.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    dtype: torch.dtype = torch.bfloat16
    max_seq_len: int = 1 << 20
    block_form: str = "sandwich"                # "sandwich" | "post_scaled" | "pre_scaled"
    residual_mult: float = 1.0                  # pre_scaled: what every sublayer's output is multiplied by
    token_side_dim: int = 0                     # pre_scaled: channels per layer of the per-layer token input (0: none)
    layer_scale: bool = False                   # pre_scaled: every sublayer's output times a per-channel ``ls1`` / ``ls2``
    norm_weight_offset: float = 0.0             # pre_scaled: norm weights are ``offset + w`` (1: stored around zero)
    logit_scale: float = 1.0
    logit_softcap: float = 0.0                  # > 0: logits <- cap * tanh(logits / cap)
    input_conv_taps: int = 0                    # post_scaled: taps of the filter in front of every sublayer
    depth_mix: bool = False                     # post_scaled: every layer hands on a mixture of all results so far

    def runs(self) -> List[Tuple[int, bool]]:
        """[(layer index, whether a repeated pass starts here)] in execution order: the layers before the span once,
        the span ``loop_times`` times, the rest once."""
        out = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            out += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, False) for i in range(self.loop_stop, len(self.layers))]


def pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Zero rows up to a multiple of 8 outputs, so that a fused projection of any width stays on the tensor-core GEMM."""
    extra = (-w.shape[0]) % multiple
    if extra == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros(extra, *w.shape[1:])], dim=0).contiguous()


class DSHybridModel(DSInferenceModelBase):
    """``weights``: ``{"embed", "final_norm_w", "unembed", "layers": [LayerWeights]}``; a layer has ``norm1``, ``norm1b``
    (+ ``norm2``, ``norm2b``, ``w_gate_up`` ``[2F, W]``, ``w_down`` with a feed-forward), ``w_in`` (the mixer's fused
    projection, rows in the order of the mixer module's ``projection layout``), ``wo``, and per kind: attention ``b_in``,
    ``sink`` (fp32); delta ``conv_w``, ``A_log``, ``dt_bias`` (fp32), ``norm``; ssd ``conv_w``, ``conv_b``, ``A_log``,
    ``dt_bias``, ``D`` (fp32), ``norm``.  Pre-scaled stacks: one norm weight per sublayer (``norm1``, ``norm2``), attention
    with filtered projections ``conv_w``, ``q_norm``, ``k_norm``, ``dist_bias`` (fp32 ``[heads, distances]``); experts
    ``moe_gate`` (fp32, the shared expert's gate row last), ``moe_gate_b``, ``moe_w1``, ``moe_w2``, ``shared_up``,
    ``shared_down``; token input ``side_gate``, ``side_proj``, ``side_norm`` and the global ``side_embed``.  With
    ``layer_scale``: ``ls1``, ``ls2``.  Channel delta rule: ``conv_w``, ``A_log``, ``dt_bias`` (fp32), ``w_a2``, ``w_g2``,
    ``norm``; latent attention ``q_norm``, ``w_uq`` (not with direct queries), ``kv_norm``, ``w_uk``, ``w_uv_t``; three-power
    feed-forward ``w_up``, ``b_up``, ``w_down``, ``b_down``, ``act_coef`` (fp32); group-limited experts ``moe_gate``,
    ``moe_correction`` (fp32), ``moe_w1``, ``moe_w2``.  Two entries of ``layers`` may be one object (borrowed weights)."""

    def __init__(self, spec: HybridSpec, weights: Dict, engine_config: RaggedInferenceEngineConfig, state_manager=None,
                 base_mp_group=None) -> None:
        super().__init__()
        if base_mp_group is not None:
            import torch.distributed as dist
            if dist.get_world_size(base_mp_group) > 1:
                raise NotImplementedError("hybrid stacks run on one tensor-parallel rank")
        self.spec = spec
        self.weights = weights
        self._engine_config = engine_config or RaggedInferenceEngineConfig()
        self.state_manager = state_manager
        self.tp_rank, self.tp_size = 0, 1
        self.flattened_params = self.flattened_param_metadata = None
        if spec.dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # exact evaluation: no reduced-precision products
            torch.backends.cudnn.allow_tf32 = False
        self._runs = spec.runs()
        # which cache / state entries every execution of a layer uses
        self._cache_of_run: Dict[int, int] = {}
        self._state_of_run: Dict[int, Tuple[int, ...]] = {}
        self._conv_of_run: Dict[int, Tuple[int, int]] = {}
        self.layer_outputs = None        # set to a list: the stream every layer run hands on is appended (a copy)
        self._build_modules()

    # ------------------------------------------------------------------------------------------ construction
    def _build_modules(self) -> None:
        s, ec = self.spec, self._engine_config
        sm = ec.state_manager
        dt, mt = DtypeEnum(s.dtype), sm.max_ragged_batch_size
        self.embed = heuristics.instantiate_embed(DSEmbeddingsConfig(
            max_tokens=mt, residual_dtype=DtypeEnum.fp32, embedding_dim=s.model_dim, scale=s.embed_scale,
            sinusoid_base=s.sinusoid_base, widen_to_residual=True), ec)
        self.norm = heuristics.instantiate_sandwich_norm(DSNormConfig(
            max_tokens=mt, type=NormTypeEnum.RMSNorm, channels=s.model_dim, residual_dtype=DtypeEnum.fp32,
            input_dtype=dt, output_dtype=dt, eps=s.norm_eps), ec)
        self.linear = heuristics.instantiate_linear(DSLinearConfig(
            max_tokens=mt, in_channels=s.model_dim, out_channels=s.model_dim, input_dtype=dt, output_dtype=dt), ec)
        if s.block_form == "post_scaled":
            self.post_norm = heuristics.instantiate_scaled_post_norm(DSNormConfig(
                max_tokens=mt, type=NormTypeEnum.RMSNorm, channels=s.model_dim, residual_dtype=DtypeEnum.fp32,
                input_dtype=dt, output_dtype=dt, eps=s.norm_eps), ec)
        elif s.block_form not in ("sandwich", "pre_scaled"):
            raise ValueError(f"unknown block form {s.block_form!r}")
        self.mixers, self.moes = [], []
        for L in s.layers:
            moe = None
            if L.ff_dim > 0 and L.ff_kind == "moe":
                moe = heuristics.instantiate_moe(DSMoEConfig(
                    max_tokens=mt, model_dim=s.model_dim, intermediate_features=L.ff_dim, n_experts=L.n_experts,
                    top_k=L.top_k, input_dtype=dt, output_dtype=dt,
                    activation=({"silu": ActivationType.SiGLU, "gelu": ActivationType.GEGLU,
                                 "relu": ActivationType.ReGLU,
                                 "clamped_swish": ActivationType.CLAMPED_SWIGLU} if L.ff_gated else
                                {"silu": ActivationType.SILU, "gelu": ActivationType.GELU, "relu": ActivationType.RELU,
                                 "relu_sq": ActivationType.RELU_SQ})[L.ff_activation],
                    normalize_scores=L.moe_renormalize,
                    score_function=L.moe_score, weight_input=L.moe_weight_input, router_dtype=DtypeEnum.fp32,
                    router_bias=L.router_bias, shared_features=L.shared_ff_dim,
                    score_correction=L.moe_correction, n_groups=L.moe_groups, keep_groups=L.moe_keep_groups,
                    score_scale=L.moe_scale, identity_experts=L.moe_identity, activation_limit=L.ff_limit), ec)
            self.moes.append(moe)
            if L.kind == "latent_attention":
                mod = heuristics.instantiate_attention(DSSelfAttentionConfig(
                    max_tokens=mt, n_heads_q=L.n_heads, n_heads_kv=1, head_size=L.key_dim, v_head_size=L.value_dim,
                    max_sequences=sm.max_ragged_sequence_count, scale_factor=L.attn_scale, input_dtype=dt,
                    output_dtype=dt,
                    masking_type=MaskingType.sliding_window if L.window > 0 else MaskingType.causal,
                    masking_args={"size": L.window} if L.window > 0 else {},
                    positional_embedding_type=(PositionalEmbeddingType.rotate_every_other if L.rot_dims > 0
                                               else PositionalEmbeddingType.none),
                    positional_embedding_config=RotateHalfConfig(theta_base=L.rot_base, rotate_dim=L.rot_dims),
                    qk_norm_eps=s.norm_eps, sink=L.sink, kv_latent_dim=L.kv_rank, rope_head_dim=L.rot_dim,
                    output_gate=L.out_gate, output_gate_per_head=L.gate_per_head, q_direct=L.q_direct,
                    rotary_scaling=None if L.rot_scaling is None else RotaryScalingConfig(
                        factor=L.rot_scaling[0], original=L.rot_scaling[1], fast=L.rot_scaling[2],
                        slow=L.rot_scaling[3])), ec)
            elif L.kind == "attention" and (L.conv_taps > 1 or L.qk_norm_weight or L.dist_rows > 0 or L.out_gate
                                            or L.q_temp_coef != 0.0):
                mask = (MaskingType.chunked if L.chunk_size > 0 else
                        MaskingType.sliding_window if L.window > 0 else MaskingType.causal)
                mod = heuristics.instantiate_attention(DSSelfAttentionConfig(
                    max_tokens=mt, n_heads_q=L.n_heads, n_heads_kv=L.n_heads_kv, head_size=L.key_dim,
                    v_head_size=L.value_dim, max_sequences=sm.max_ragged_sequence_count, scale_factor=L.attn_scale,
                    input_dtype=dt, output_dtype=dt, masking_type=mask,
                    masking_args={"size": L.chunk_size or L.window} if mask != MaskingType.causal else {},
                    positional_embedding_type=(PositionalEmbeddingType.distance_bias if L.dist_rows > 0
                                               else PositionalEmbeddingType.none),
                    distance_bias=DistanceBiasConfig(rows=L.dist_rows, far=L.dist_far) if L.dist_rows > 0 else None,
                    qk_norm_eps=s.norm_eps, qkv_conv_taps=L.conv_taps, qk_norm_weight=L.qk_norm_weight,
                    q_temp_coef=L.q_temp_coef, q_temp_every=L.q_temp_every, output_gate=L.out_gate), ec)
            elif L.kind == "attention":
                mod = heuristics.instantiate_attention(DSSelfAttentionConfig(
                    max_tokens=mt, n_heads_q=L.n_heads, n_heads_kv=L.n_heads_kv, head_size=L.key_dim,
                    v_head_size=L.value_dim, max_sequences=sm.max_ragged_sequence_count, scale_factor=L.attn_scale,
                    input_dtype=dt, output_dtype=dt,
                    masking_type=MaskingType.chunked if L.chunk_size > 0 else MaskingType.causal,
                    masking_args={"size": L.chunk_size} if L.chunk_size > 0 else {},
                    positional_embedding_type=PositionalEmbeddingType.none, qk_unit_rms=L.qk_unit_rms,
                    qk_norm_eps=s.norm_eps, sink=L.sink), ec)
            else:
                mod = heuristics.instantiate_recurrent_mixer(DSRecurrentMixerConfig(
                    max_tokens=mt, kind=L.kind, model_dim=s.model_dim, n_heads=L.n_heads, n_heads_kv=L.n_heads_kv,
                    key_dim=L.key_dim, value_dim=L.value_dim, conv_taps=L.conv_taps, norm_groups=L.norm_groups,
                    gate_cap=L.gate_cap, eps=s.norm_eps, max_sequences=sm.max_ragged_sequence_count, input_dtype=dt, output_dtype=dt), ec)
            self.mixers.append(mod)
        n_cache = 0
        self._state_cfg = StatePoolConfig()
        shapes = []
        for r, (li, _) in enumerate(self._runs):
            L = s.layers[li]
            if L.kind == "attention":
                self._cache_of_run[r] = n_cache
                shapes.append((L.n_heads_kv, L.key_dim, L.value_dim))
                n_cache += 1
                if hasattr(self.mixers[li], "state_shapes"):        # carried inputs of filtered projections
                    self._state_of_run[r] = tuple(self._state_cfg.add(shape, sdt)
                                                  for shape, sdt in self.mixers[li].state_shapes())
            elif L.kind == "latent_attention":
                self._cache_of_run[r] = n_cache
                shapes.append((1, self.mixers[li].cache_row, 0))        # latent | rotated key part; no value tensor
                n_cache += 1
            else:
                self._state_of_run[r] = tuple(self._state_cfg.add(shape, sdt)
                                              for shape, sdt in self.mixers[li].state_shapes())
            if s.block_form == "post_scaled":
                # the last taps - 1 inputs of the filter in front of the mixer and of the one in front of the feed-forward
                keep = (max(s.input_conv_taps, 1) - 1, s.model_dim)
                self._conv_of_run[r] = (self._state_cfg.add(keep, torch.float32),
                                        self._state_cfg.add(keep, torch.float32) if L.ff_dim > 0 else -1)
        self._cache_shapes = tuple(shapes)
        self._stack = None

    # ------------------------------------------------------------------------------------------ properties
    @property
    def num_layers(self): return len(self.spec.layers)
    @property
    def model_dim(self): return self.spec.model_dim
    @property
    def vocab_size(self): return self.spec.vocab_size
    @property
    def activation_dtype(self): return DtypeEnum(self.spec.dtype)
    @property
    def max_sequence_length(self): return self.spec.max_seq_len

    # ------------------------------------------------------------------------------------------ memory planning
    def kv_cache_config(self, block_size: int) -> KVCacheConfig:
        """One (keys, values) pair per EXECUTION of an attention layer: a repeated layer keeps a cache per pass."""
        return KVCacheConfig(block_size=block_size, cache_shape=(len(self._cache_shapes), 1, 1),
                             cache_dtype=self.spec.dtype, layer_shapes=self._cache_shapes)

    def state_pool_config(self) -> StatePoolConfig:
        """Carried convolution inputs and matrix state per execution of a recurrent layer."""
        return self._state_cfg

    def get_kv_requirements(self, sequence, max_new_tokens: int, max_new_blocks: int):
        bs = self.state_manager.kv_block_size
        total = sequence.seen_tokens + max_new_tokens
        need = ceil_div(total, bs) - sequence.cur_allocated_blocks
        if need > max_new_blocks:
            fit = (sequence.cur_allocated_blocks + max_new_blocks) * bs - sequence.seen_tokens
            return max(0, fit), max_new_blocks
        return max_new_tokens, max(0, need)

    def get_remaining_block_capacity(self, sequence) -> int:
        return sequence.cur_allocated_blocks * self.state_manager.kv_block_size - sequence.seen_tokens

    def maybe_allocate_kv(self, sequence, n_new_tokens: int) -> None:
        _, need = self.get_kv_requirements(sequence, n_new_tokens, self.state_manager.free_blocks)
        if need > 0:
            sequence.extend_kv_cache(self.state_manager.allocate_blocks(need))

    def maybe_free_kv(self, sequence) -> None:
        """Chunk-local layers could return the pages before the current chunk; every page is kept."""

    # ------------------------------------------------------------------------------------------ forward
    def _feed_forward(self, L: HybridLayerSpec, lw: LayerWeights, x: torch.Tensor, li: int = -1) -> torch.Tensor:
        if L.ff_kind == "moe":
            if L.moe_correction or L.moe_identity > 0:
                return self.moes[li](x, lw.moe_gate, lw.moe_w1, lw.moe_w2,
                                     correction=lw.moe_correction if L.moe_correction else None)
            if L.router_bias or L.shared_ff_dim > 0:
                return self.moes[li](x, lw.moe_gate, lw.moe_w1, lw.moe_w2, gate_b=lw.moe_gate_b if L.router_bias else None,
                                     shared=(lw.shared_up, lw.shared_down) if L.shared_ff_dim > 0 else None)
            return self.moes[li](x, lw.moe_gate, lw.moe_w1, lw.moe_w2)
        if L.ff_kind == "biased":
            if L.ff_activation == "power_norm":
                h = M.power_norm_act(self.linear(x, lw.w_up), lw.b_up, lw.act_coef, self.spec.norm_eps)
            else:
                h = M.bias_act_rows(self.linear(x, lw.w_up), lw.b_up, L.ff_activation)
            return F.linear(h, lw.w_down, lw.b_down)
        h = self.linear(x, lw.w_gate_up)
        if h.is_cuda and h.dtype == torch.bfloat16 and L.ff_dim % 8 == 0:
            h = F.gated_act(h, L.ff_activation)
        else:
            h = M.gated_act_rows(h, L.ff_activation)
        return self.linear(h, lw.w_down)

    def _mixer(self, r: int, li: int, lw: LayerWeights, x: torch.Tensor, batch) -> torch.Tensor:
        L, mod, sm = self.spec.layers[li], self.mixers[li], self.state_manager
        proj = self.linear(x, lw.w_in)
        if L.kind == "attention" and hasattr(mod, "filtered_channels"):
            states = self._state_of_run.get(r, ())
            ctx = mod(proj, sm.get_cache(self._cache_of_run[r]), batch, None, lw,
                      sm.get_state(states[0]) if states else None)
        elif L.kind == "attention":
            ctx = mod(proj, sm.get_cache(self._cache_of_run[r]), batch, None, lw.b_in, lw.sink)
        elif L.kind == "latent_attention":
            ctx = mod(proj, sm.get_cache(self._cache_of_run[r]), batch, None, lw)
        else:
            ctx = mod(proj, lw, tuple(sm.get_state(e) for e in self._state_of_run[r]), batch)
        return self.linear(ctx, lw.wo)

    def _filtered(self, x: torch.Tensor, w: torch.Tensor, entry: int, batch) -> torch.Tensor:
        """What a sublayer of a post-scaled layer reads: ``x + filter(x)`` in the activation dtype; the sequence's
        carried inputs move on by this batch's rows."""
        state = self.state_manager.get_state(entry)
        h = M.conv_residual(x, w, state, batch.seq_info(), batch.token_to_seq(), self.spec.dtype)
        M.conv_state_update(x, state, batch.seq_info())
        return h

    @torch.no_grad()
    def _forward_post_scaled(self, batch) -> torch.Tensor:
        """Layers ``x <- x + ls1 (.) norm1(mixer(x + conv1(x)))``, ``x <- x + ls2 (.) norm2(ff(x + conv2(x)))``; with
        ``depth_mix`` layer ``i`` hands on ``sum_j mix[j] X_j`` over the embedding ``X_0`` and the results ``X_1 ..
        X_(i+1)`` of the layers so far, which are kept as a stack of fp32 streams for the length of the forward."""
        W, s = self.weights, self.spec
        T = batch.current_tokens
        n_runs = len(self._runs)
        x = self.embed(batch, W["embed"])
        if s.depth_mix:
            if self._stack is None or self._stack.shape[1] < T:
                self._stack = torch.empty(n_runs + 1, max(T, 1), s.model_dim, dtype=torch.float32, device=x.device)
            stack = self._stack[:, :T]
            stack[0].copy_(x)
        for r, (li, _) in enumerate(self._runs):
            lw, L = W["layers"][li], s.layers[li]
            c1, c2 = self._conv_of_run[r]
            y = self._mixer(r, li, lw, self._filtered(x, lw.conv1, c1, batch), batch)
            last = L.ff_dim == 0
            mid = torch.empty_like(x)

            def close(x_in, y, gain, scale, final):
                if not final:
                    return self.post_norm(x_in, y, gain, None, scale, mid)
                if not s.depth_mix:
                    return self.post_norm(x_in, y, gain, None, scale, mid)
                nxt = torch.empty_like(x_in)
                self.post_norm(x_in, y, gain, None, scale, stack[r + 1], (stack, r + 1, lw.depth_mix, nxt))
                return nxt
            x = close(x, y, lw.norm1, lw.ls1, last)
            if not last:
                y = self._feed_forward(L, lw, self._filtered(x, lw.conv2, c2, batch), li)
                x = close(x, y, lw.norm2, lw.ls2, True)
            if self.layer_outputs is not None:
                self.layer_outputs.append(x.clone())
        rows = batch.last_token_index()
        if rows.numel() == 0:               # a step that only advances caches and states
            return torch.empty(0, s.vocab_size, dtype=torch.float32, device=x.device)
        h = M.rms_scale_rows(x, rows, W["final_norm_w"], s.norm_eps, s.dtype)
        return self.linear(h, W["unembed"])[:, : s.vocab_size].float()

    def _token_side(self, li: int, lw: LayerWeights, x: torch.Tensor, batch) -> torch.Tensor:
        """Per-layer token input, before its norm: ``proj(gelu(gate x) * e)`` with ``e`` the layer's ``token_side_dim``
        channels of the token's row of the side table; ``x`` is the stream in the activation dtype."""
        s = self.spec
        gx = self.linear(x, lw.side_gate)
        g = M.side_gate(gx, self.weights["side_embed"], batch.input_ids(), li * s.token_side_dim, s.token_side_dim,
                        lw.side_proj.shape[1])
        return self.linear(g, lw.side_proj)

    @torch.no_grad()
    def _forward_pre_scaled(self, batch) -> torch.Tensor:
        """Layers ``x <- x + m mixer(norm1(x))``, ``x <- x + m ff(norm2(x))``, ``x <- x + m rms_norm(side(x)) w``.  The
        output of a sublayer is added by the kernel that also computes what the next sublayer reads (its norm, or the
        stream itself in the activation dtype for the token input), so ``y`` below is always one addition behind."""
        W, s = self.weights, self.spec
        m, off = s.residual_mult, s.norm_weight_offset
        resid = self.embed(batch, W["embed"])
        first = resid.clone() if any(again for _, again in self._runs) else None
        y = post = ls = None            # pending: resid += m * ls (.) y (post None) or m * ls (.) rms_norm(y) * post
        for r, (li, again) in enumerate(self._runs):
            lw, L = W["layers"][li], s.layers[li]
            _, x = self.norm(resid, y, lw.norm1, None, post, first if again else None, m, False, ls, off)
            y, post, ls = self._mixer(r, li, lw, x, batch), None, lw.ls1 if s.layer_scale else None
            if L.ff_dim > 0:
                _, x = self.norm(resid, y, lw.norm2, None, None, None, m, False, ls, off)
                y, ls = self._feed_forward(L, lw, x, li), lw.ls2 if s.layer_scale else None
            if s.token_side_dim > 0:
                _, x = self.norm(resid, y, None, None, None, None, m, True, ls)
                y, post, ls = self._token_side(li, lw, x, batch), lw.side_norm, None
            if self.layer_outputs is not None:
                self.norm(resid, y, None, None, post, None, m, False, ls)
                y = post = ls = None
                self.layer_outputs.append(resid.clone())
        rows = batch.last_token_index().long()
        if rows.numel() == 0:               # a step that only advances caches and states
            return torch.empty(0, s.vocab_size, dtype=torch.float32, device=resid.device)
        resid = resid.index_select(0, rows)
        _, x = self.norm(resid, None if y is None else y.index_select(0, rows), W["final_norm_w"], None, post, None, m,
                         False, ls, off)
        logits = self.linear(x, W["unembed"])[:, : s.vocab_size].float().contiguous()
        if s.logit_scale != 1.0 or s.logit_softcap > 0.0:
            M.scale_softcap_(logits, s.logit_scale, s.logit_softcap)
        return logits

    @torch.no_grad()
    def forward(self, batch) -> torch.Tensor:
        W, s = self.weights, self.spec
        if s.block_form == "post_scaled":
            return self._forward_post_scaled(batch)
        if s.block_form == "pre_scaled":
            return self._forward_pre_scaled(batch)
        resid = self.embed(batch, W["embed"])
        first = resid.clone() if any(again for _, again in self._runs) else None
        y = post = None                     # output of the last sublayer and its post-norm weight, not yet added
        for r, (li, again) in enumerate(self._runs):
            lw, L = W["layers"][li], s.layers[li]
            _, x = self.norm(resid, y, lw.norm1, None, post, first if again else None)
            y, post = self._mixer(r, li, lw, x, batch), lw.norm1b
            if L.ff_dim > 0:
                _, x = self.norm(resid, y, lw.norm2, None, post, None)
                y, post = self._feed_forward(L, lw, x, li), lw.norm2b
        rows = batch.last_token_index().long()
        if rows.numel() == 0:               # a step that only advances caches and states
            return torch.empty(0, s.vocab_size, dtype=torch.float32, device=resid.device)
        resid = resid.index_select(0, rows)
        _, x = self.norm(resid, None if y is None else y.index_select(0, rows), W["final_norm_w"], None, post, None)
        return self.linear(x, W["unembed"])[:, : s.vocab_size].float()
