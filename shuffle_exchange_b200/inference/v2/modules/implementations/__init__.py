"""Concrete module implementations on the framework's sm_100a kernels (reference
``inference/v2/modules/implementations/{attention,embedding,linear,moe,pre_norm,post_norm,unembed}/*``).

=========================  =======================================================================================
 ``dense_blocked_attention``  ``sxb_kv_rotary_blocked`` (rotary + paged-cache append) + ``sxb_paged_attention``
 ``ragged_embedding``         ``sxb_ragged_embed`` (token + optional positional table with offset)
 ``blas_fp_linear``           tcgen05 GEMM + fused bias/activation or gated activation
 ``quantized_wf6af16_linear`` weights stored FP6 (group-scaled), dequantised to bf16 per call, tcgen05 GEMM
 ``cutlass_multi_gemm_moe``   top-k gating / scatter / per-expert GEMMs over contiguous row ranges / weighted gather
 ``cuda_pre_ln / cuda_pre_rms / cuda_post_ln``   fused residual-add + norm kernels
 ``ragged_unembed``           (norm +) last-token gather + vocabulary GEMM
 ``sink_chunked_attention``   bias + unit-RMS q/k + cache append (``sxb_qk_norm_append``), causal or chunk-local softmax
                              with a sink logit over the paged cache in fp32 (``sxb_sink_attention``)
 ``scaled_sinusoid_embedding``  token row * scale (+ sinusoidal position vector) into an fp32 residual
 ``latent_sink_attention``    keys / values as up-projections of one cached latent per token (+ a shared rotated key
                              part); attention in the latent space, sliding window, sink logit
 ``mlstm_mixer``              matrix-memory LSTM: exponential gating with a running maximum around the linear recurrence
 ``fp32_scaled_post_rms``     fp32 stream += scale (.) rms_norm(sublayer output) * gain (+ mixture of all layers' streams)
 ``fp32_sandwich_rms``        fp32 residual += post-norm(sublayer output); next pre-norm, one kernel
 ``filtered_bias_attention``  q | k | v through a short causal filter with carried inputs, weighted per-head RMS norm,
                              query temperature, learned distance-bucket bias on the scores, sigmoid output gate
 ``gated_delta_mixer`` / ``ssd_mixer``   short convolutions with carried inputs + linear recurrence with a matrix
                              state per (sequence slot, head) + gated group norm
 ``channel_delta_mixer``      the delta rule with a separate decay for every key channel of every head and a sigmoid output gate, both
                              from two-step projections
=========================  =======================================================================================
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch

from .....ops import functional as F
from .....ops import moe_ops
from ...inference_parameter import InferenceParameter
from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum, is_gated
from ...kernels import ragged_ops as R
from ...kernels import mixer_ops as M
from ..configs import (DSEmbeddingsConfig, DSLinearConfig, DSMoEConfig, DSNormConfig, DSRecurrentMixerConfig,
                       DSSelfAttentionConfig, DSUnembedConfig, MaskingType, PositionalEmbeddingType)
from ..interfaces import (DSEmbeddingBase, DSEmbeddingRegistry, DSLinearBase, DSLinearRegistry, DSMoEBase,
                          DSMoERegistry, DSPostNormBase, DSPostNormRegistry, DSPreNormBase, DSPreNormRegistry,
                          DSRecurrentMixerBase, DSRecurrentMixerRegistry, DSSelfAttentionBase, DSSelfAttentionRegistry,
                          DSUnembedBase, DSUnembedRegistry, _param)


def _dt(x) -> DtypeEnum:
    """Config models may store enum members by value: normalise."""
    return x if isinstance(x, DtypeEnum) else DtypeEnum(x)


def _act_name(act: ActivationType) -> str:
    return {ActivationType.GELU: "gelu", ActivationType.RELU: "relu", ActivationType.SILU: "silu",
            ActivationType.GEGLU: "gelu", ActivationType.ReGLU: "relu", ActivationType.SiGLU: "silu",
            ActivationType.IDENTITY: "identity", ActivationType.RELU_SQ: "relu_sq",
            ActivationType.CLAMPED_SWIGLU: "clamped_swish"}[ActivationType(act)]


def _apply_activation(y: torch.Tensor, bias: Optional[torch.Tensor], act: ActivationType, limit: float = 0.0) -> torch.Tensor:
    act = ActivationType(act)
    if is_gated(act):
        # fused weights are [gate | up] halves (HF gate_proj / up_proj order): act(gate) * up
        if bias is not None:
            y = y + bias
        if act == ActivationType.CLAMPED_SWIGLU:
            return M.gated_act_rows(y, "clamped_swish", limit)
        if y.is_cuda and (y.dtype != torch.bfloat16 or (y.shape[-1] // 2) % 8):
            return M.gated_act_rows(y, _act_name(act))       # fp32 rows, or halves that are not 16-byte multiples
        return F.gated_act(y, _act_name(act))
    if act == ActivationType.IDENTITY:
        return y if bias is None else y + bias
    if act == ActivationType.RELU_SQ or (y.is_cuda and y.dtype == torch.float32):
        return M.bias_act_rows(y, bias, _act_name(act))
    return F.bias_act(y, bias, _act_name(act))


# ============================================================================================ attention
@DSSelfAttentionRegistry.register_module
class DSDenseBlockedAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "dense_blocked_attention"

    @staticmethod
    def supports_config(config: DSSelfAttentionConfig) -> bool:
        if MaskingType(config.masking_type) != MaskingType.causal:
            return False
        if config.sink or config.qk_unit_rms or config.v_head_size not in (None, config.head_size):
            return False
        return PositionalEmbeddingType(config.positional_embedding_type) in (PositionalEmbeddingType.none,
                                                                             PositionalEmbeddingType.rotate_half)

    def __init__(self, config: DSSelfAttentionConfig, implementation_config: Dict[str, Any]) -> None:
        super().__init__(config, implementation_config)
        rot = config.positional_embedding_config
        if PositionalEmbeddingType(config.positional_embedding_type) == PositionalEmbeddingType.rotate_half:
            self._rot_dim = config.head_size if rot is None or rot.rotate_dim is None else rot.rotate_dim
            self._theta = 10000.0 if rot is None else rot.theta_base
        else:
            self._rot_dim, self._theta = 0, 10000.0

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 128

    def forward(self, q_k_v: torch.Tensor, kv_cache: torch.Tensor, batch, inv_freqs=None) -> torch.Tensor:
        c = self._config
        t2s, pos, tables = batch.token_to_seq(), batch.token_positions(), batch.block_tables()
        R.kv_rotary_blocked(q_k_v, kv_cache, t2s, pos, tables, c.n_heads_q, c.n_heads_kv, c.head_size, self._rot_dim,
                            self._theta)
        q = q_k_v.view(q_k_v.shape[0], c.n_heads_q + 2 * c.n_heads_kv, c.head_size)[:, :c.n_heads_q]
        out = R.ragged_attention(q, kv_cache, batch, scale=c.scale_factor)
        return out.reshape(out.shape[0], c.n_heads_q * c.head_size)


# ============================================================================================ embedding
@DSEmbeddingRegistry.register_module
class DSRaggedEmbedding(DSEmbeddingBase):

    @staticmethod
    def name() -> str:
        return "ragged_embedding"

    @staticmethod
    def supports_config(config: DSEmbeddingsConfig) -> bool:
        return (not config.use_token_type and config.output_normalization is None and config.sinusoid_base is None
                and config.scale == 1.0)

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def forward(self, ragged_batch, word_embeddings, position_embeddings=None, token_type_ids=None,
                token_type_embeddings=None) -> torch.Tensor:
        ids = ragged_batch.input_ids()
        if self._config.positional_embedding:
            self._output = R.ragged_embed(ids, word_embeddings, ragged_batch.token_positions(), position_embeddings,
                                          self._config.positional_offset)
        else:
            self._output = R.ragged_embed(ids, word_embeddings)
        return self._output


# ============================================================================================ linear
@DSLinearRegistry.register_module
class BlasFPLinear(DSLinearBase):

    @staticmethod
    def name() -> str:
        return "blas_fp_linear"

    @staticmethod
    def supports_config(config: DSLinearConfig) -> bool:
        return _dt(config.input_dtype) == _dt(config.output_dtype) and _dt(config.input_dtype) in (
            DtypeEnum.fp16, DtypeEnum.bf16, DtypeEnum.fp32)

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None

    def transform_param(self, param: torch.Tensor) -> InferenceParameter:
        return _param(param.to(_dt(self._config.input_dtype).torch))

    def forward(self, hidden_states, w, b=None) -> torch.Tensor:
        self._output = _apply_activation(F.linear(hidden_states, w), b, self._config.activation)
        return self._output

    @property
    def output(self) -> torch.Tensor:
        return self._output


@DSLinearRegistry.register_module
class QuantizedWf6Af16Linear(DSLinearBase):
    """FP6 (e3m2, group-scaled) weights, 16-bit activations — the reference's ``cuda_linear`` W6A16 path
    (``kernels/core_ops/cuda_linear``).  Weights cost 6 bits + scales in HBM; each call dequantises the layer into a
    bf16 scratch and runs the tcgen05 GEMM (decode GEMMs are weight-bandwidth bound: 2.6x less weight traffic)."""

    GROUP = 512

    @staticmethod
    def name() -> str:
        return "quantized_wf6af16_linear"

    @staticmethod
    def supports_config(config: DSLinearConfig) -> bool:
        return _dt(config.input_dtype) == _dt(config.output_dtype) and _dt(config.input_dtype) in (
            DtypeEnum.fp16, DtypeEnum.bf16) and config.in_channels % 64 == 0 and config.out_channels % 256 == 0

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None
        from .....ops.fp_quantizer import FP_Quantize
        self._q = FP_Quantize(group_size=self.GROUP)

    def transform_param(self, param: torch.Tensor) -> InferenceParameter:
        if param.dim() == 1:
            return _param(param.to(_dt(self._config.input_dtype).torch))
        w = param.to(torch.bfloat16).contiguous()
        if w.numel() % self.GROUP != 0:
            return _param(w)
        q = self._q.quantize(w, q_bits=6, q_mantisa_bits=2, return_meta_tensor=False)
        return InferenceParameter.initialize(q, shape_marker=torch.tensor(list(w.shape)))

    def forward(self, hidden_states, w, b=None) -> torch.Tensor:
        if w.dtype == torch.uint8:
            shape = tuple(int(s) for s in w.shape_marker.tolist())
            dense = self._q.dequantize(w, fp_out=torch.empty(shape, dtype=torch.bfloat16, device=w.device), q_bits=6,
                                       q_mantisa_bits=2).view(shape)
        else:
            dense = w
        self._output = _apply_activation(F.linear(hidden_states, dense.to(hidden_states.dtype)), b,
                                         self._config.activation)
        return self._output

    @property
    def output(self) -> torch.Tensor:
        return self._output


# ============================================================================================ MoE
@DSMoERegistry.register_module
class DSMultiGemmMoE(DSMoEBase):

    @staticmethod
    def name() -> str:
        return "cutlass_multi_gemm_moe"

    @staticmethod
    def supports_config(config: DSMoEConfig) -> bool:
        return (_dt(config.input_dtype) == _dt(config.output_dtype) and 1 <= config.top_k <= 8
                and config.top_k <= config.n_experts + config.identity_experts
                and config.score_function in ("softmax", "sigmoid"))

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None

    def transform_gate_param(self, param):
        return _param(param.to(_dt(self._config.input_dtype).torch))

    def transform_moe_mlp_1_param(self, param):
        return _param(param.to(_dt(self._config.input_dtype).torch))      # [E, (1|2) * F, H]

    def transform_moe_mlp_2_param(self, param):
        return _param(param.to(_dt(self._config.input_dtype).torch))      # [E, H, F]

    def _shared(self, out, hidden_states, gate_logit, shared):
        """``out += sigmoid(gate_logit) * down(act(up(h)))``: the expert every token uses."""
        w_up, w_down = shared
        h = _apply_activation(F.linear(hidden_states, w_up), None, self._config.activation)
        return M.row_gate_add_(out, F.linear(h, w_down)[:, : out.shape[1]].contiguous(), gate_logit)

    def forward(self, hidden_states, gate_w, mlp_1_w, mlp_2_w, mlp_1_b=None, mlp_2_b=None, gate_b=None,
                shared=None, correction=None) -> torch.Tensor:
        """``gate_w`` ``[E (+ 1), H]``: the experts' router rows and, with ``shared_features``, one more row whose logit
        gates the shared expert ``shared = (w_up [Fs, H], w_down [H, Fs])``; ``gate_b`` the logits' bias.  With
        ``identity_experts`` the router has ``E + identity_experts`` rows (the identity experts last) and
        ``correction`` (fp32, one per router row) is added to the scores for the choice only."""
        c = self._config
        if c.router_dtype is not None and _dt(c.router_dtype) == DtypeEnum.fp32 and gate_w.dtype == torch.float32:
            logits = M.router_logits(hidden_states, gate_w, gate_b)       # 32-bit product straight from the 16-bit rows
        elif c.router_dtype is not None and _dt(c.router_dtype).torch != hidden_states.dtype:
            rd = _dt(c.router_dtype).torch
            logits = torch.nn.functional.linear(hidden_states.to(rd), gate_w.to(rd), gate_b)
        else:
            logits = torch.nn.functional.linear(hidden_states, gate_w, gate_b)
        shared_logit = None
        if c.shared_features > 0:
            shared_logit = logits[:, c.n_experts].float()
            logits = logits[:, : c.n_experts].contiguous()
        out = self._routed(hidden_states, logits, mlp_1_w, mlp_2_w, mlp_1_b, mlp_2_b, correction)
        if shared_logit is not None:
            out = self._shared(out, hidden_states, shared_logit, shared)
        self._output = out
        return out

    def _routed(self, hidden_states, logits, mlp_1_w, mlp_2_w, mlp_1_b, mlp_2_b, correction=None) -> torch.Tensor:
        c = self._config
        n_id = c.identity_experts
        if logits.shape[1] != c.n_experts + n_id:
            raise ValueError(f"the router has {logits.shape[1]} outputs for {c.n_experts} experts and {n_id} identity experts")
        if c.score_correction or c.n_groups > 1 or c.score_scale != 1.0 or n_id > 0:
            scores, assign, offsets, counts = moe_ops.top_k_gating(
                logits, c.top_k, score_function=c.score_function, correction=correction if c.score_correction else None,
                n_groups=c.n_groups, keep_groups=c.keep_groups, scale=c.score_scale)
        else:
            scores, assign, offsets, counts = moe_ops.top_k_gating(logits, c.top_k, renormalize=c.normalize_scores,
                                                                   score_function=c.score_function)
        from .....moe import fused_ep
        if fused_ep.grouped_inference_ok(hidden_states, mlp_1_w, mlp_2_w, mlp_1_b, mlp_2_b):
            # one grouped tcgen05 GEMM per projection over expert-contiguous rows, no host synchronisation
            self._output = fused_ep.grouped_experts_inference(
                hidden_states, scores, assign, offsets, counts, mlp_1_w, mlp_2_w,
                lambda t: _apply_activation(t, None, c.activation, c.activation_limit), c.top_k,
                weight_input=c.weight_input, n_identity=n_id)
            return self._output
        if c.weight_input:
            moe_in, cumsum, slots = moe_ops.moe_scatter_scaled(hidden_states, scores, assign, offsets, counts)
            scores = None                   # the outputs are summed as they are
        else:
            moe_in, cumsum, slots = moe_ops.moe_scatter(hidden_states, assign, offsets, counts)
        out = torch.empty_like(moe_in)
        lo = 0
        for e, hi in enumerate(cumsum.tolist()):
            if hi > lo and e >= c.n_experts:          # an identity expert hands its rows on
                out[lo:hi] = moe_in[lo:hi]
            elif hi > lo:
                h = _apply_activation(F.linear(moe_in[lo:hi], mlp_1_w[e]),
                                      None if mlp_1_b is None else mlp_1_b[e], c.activation, c.activation_limit)
                y = F.linear(h, mlp_2_w[e])
                out[lo:hi] = y if mlp_2_b is None else y + mlp_2_b[e]
            lo = hi
        self._output = moe_ops.moe_gather(out, scores, slots)
        return self._output

    @property
    def output(self) -> torch.Tensor:
        return self._output


# ============================================================================================ norms
def _norm(cfg: DSNormConfig, x, gamma, beta, residual=None):
    if NormTypeEnum(cfg.type) == NormTypeEnum.RMSNorm:
        return F.rms_norm(x, gamma, cfg.eps, residual)
    return F.layer_norm(x, gamma, beta, cfg.eps, residual)


@DSPreNormRegistry.register_module
class DSPreLNCUDAModule(DSPreNormBase):

    @staticmethod
    def name() -> str:
        return "cuda_pre_ln"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return NormTypeEnum(config.type) == NormTypeEnum.LayerNorm

    def forward(self, residual, hidden_states, gamma, beta=None) -> Tuple[torch.Tensor, torch.Tensor]:
        if hidden_states is None:
            return residual, _norm(self._config, residual, gamma, beta)[0]
        y, res = _norm(self._config, hidden_states, gamma, beta, residual)
        return res, y


@DSPreNormRegistry.register_module
class DSPreRMSCUDAModule(DSPreLNCUDAModule):

    @staticmethod
    def name() -> str:
        return "cuda_pre_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return NormTypeEnum(config.type) == NormTypeEnum.RMSNorm


@DSPostNormRegistry.register_module
class DSPostLNCUDAModule(DSPostNormBase):

    @staticmethod
    def name() -> str:
        return "cuda_post_ln"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return NormTypeEnum(config.type) == NormTypeEnum.LayerNorm

    def forward(self, residual, hidden_states, gamma, beta=None) -> torch.Tensor:
        return _norm(self._config, hidden_states, gamma, beta, residual)[0]


# ============================================================================================ unembed
@DSUnembedRegistry.register_module
class DSRaggedUnembed(DSUnembedBase):

    @staticmethod
    def name() -> str:
        return "ragged_unembed"

    @staticmethod
    def supports_config(config: DSUnembedConfig) -> bool:
        return True

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def forward(self, hidden_states, vocab_embedding, ragged_metadata, bias=None, gamma=None, beta=None):
        c = self._config
        last = R.logits_gather(hidden_states, ragged_metadata.last_token_index())
        if c.norm_type is not None and gamma is not None:
            if NormTypeEnum(c.norm_type) == NormTypeEnum.RMSNorm:
                last = F.rms_norm(last, gamma, c.eps)[0]
            else:
                last = F.layer_norm(last, gamma, beta, c.eps)[0]
        logits = F.linear(last, vocab_embedding)
        self._output = logits if bias is None else logits + bias
        return self._output


# ============================================================================================ hybrid stacks
@DSSelfAttentionRegistry.register_module
class DSSinkChunkedAttention(DSSelfAttentionBase):
    """Attention without rotation whose value heads may be narrower than its key heads: optional per-head unit-RMS
    of q and k, causal or chunk-local mask, optional sink logit in the softmax denominator.  Scores, weights and the
    weighted sum are fp32; the paged cache is a ``(keys, values)`` pair in the activation dtype."""

    @staticmethod
    def name() -> str:
        return "sink_chunked_attention"

    @staticmethod
    def supports_config(config: DSSelfAttentionConfig) -> bool:
        if MaskingType(config.masking_type) not in (MaskingType.causal, MaskingType.chunked):
            return False
        if MaskingType(config.masking_type) == MaskingType.chunked and int(config.masking_args.get("size", 0)) < 1:
            return False
        if config.qkv_conv_taps > 1 or config.qk_norm_weight or config.q_temp_coef != 0.0 or config.output_gate:
            return False
        return (PositionalEmbeddingType(config.positional_embedding_type) == PositionalEmbeddingType.none
                and (config.v_head_size or config.head_size) <= 256 and config.n_heads_q % config.n_heads_kv == 0)

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    def forward(self, q_k_v: torch.Tensor, kv_cache, batch, inv_freqs=None, bias=None, sink=None) -> torch.Tensor:
        c = self._config
        dv = c.v_head_size or c.head_size
        chunk = int(c.masking_args["size"]) if MaskingType(c.masking_type) == MaskingType.chunked else 0
        keys, values = kv_cache
        t2s, pos, tables = batch.token_to_seq(), batch.token_positions(), batch.block_tables()
        q = M.qk_norm_append(q_k_v, bias, keys, values, t2s, pos, tables, c.n_heads_q, c.n_heads_kv, c.head_size, dv,
                             c.qk_norm_eps, c.qk_unit_rms)
        atoms, n_long = None, 0
        if q.is_cuda and M.tiles_supported(c.head_size, dv) and hasattr(batch, "atoms_longer_than"):
            atoms, n_long = batch.atoms(), batch.atoms_longer_than(M.SHORT_ATOM)
        return M.sink_attention(q, keys, values, sink if c.sink else None, t2s, pos, tables, c.scale_factor, chunk,
                                _dt(c.output_dtype).torch, atoms, n_long)


@DSEmbeddingRegistry.register_module
class DSScaledSinusoidEmbedding(DSEmbeddingBase):

    @staticmethod
    def name() -> str:
        return "scaled_sinusoid_embedding"

    @staticmethod
    def supports_config(config: DSEmbeddingsConfig) -> bool:
        return (not config.use_token_type and not config.positional_embedding
                and _dt(config.residual_dtype) == DtypeEnum.fp32)

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)
        self._output = None

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def forward(self, ragged_batch, word_embeddings, position_embeddings=None, token_type_ids=None,
                token_type_embeddings=None) -> torch.Tensor:
        c = self._config
        self._output = M.embed_sinusoid(ragged_batch.input_ids(), ragged_batch.token_positions(), word_embeddings,
                                        c.scale, c.sinusoid_base)
        return self._output


@DSPreNormRegistry.register_module
class DSSandwichRMSNorm(DSPreNormBase):
    """Layers of the form ``x <- x + post_norm(sublayer(pre_norm(x)))`` on an fp32 residual: one kernel closes the
    previous sublayer (``residual += mult * rms_norm(hidden) * gamma_post``; without ``gamma_post`` the sublayer has no
    post-norm: ``residual += mult * hidden``), optionally adds another fp32 stream, and opens the next one (returns
    ``rms_norm(residual) * gamma``; without ``gamma``: the stream itself in the output dtype if ``copy_out``)."""

    @staticmethod
    def name() -> str:
        return "fp32_sandwich_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return NormTypeEnum(config.type) == NormTypeEnum.RMSNorm and _dt(config.residual_dtype) == DtypeEnum.fp32

    def forward(self, residual, hidden_states, gamma, beta=None, gamma_post=None, extra=None, mult=1.0, copy_out=False,
                channel_scale=None, gamma_offset=0.0):
        """``channel_scale`` ``[W]``: what the closed sublayer adds is also multiplied per channel (a layer scale);
        ``gamma_offset``: the opening norm's weight is ``gamma_offset + gamma`` (1 for weights stored around zero)."""
        y = M.resid_norm_step(residual, hidden_states, gamma_post, extra, gamma, self._config.eps,
                              _dt(self._config.output_dtype).torch, mult, copy_out, channel_scale, gamma_offset)
        return residual, y


class _RecurrentMixer(DSRecurrentMixerBase):

    def __init__(self, config, implementation_config):
        super().__init__(config, implementation_config)

    @property
    def conv_channels(self) -> int:
        raise NotImplementedError

    def state_shapes(self):
        """[(shape per sequence, dtype)]: the convolution's carried inputs, then the matrix state of every head."""
        c = self._config
        return [((c.conv_taps - 1, self.conv_channels), _dt(c.input_dtype).torch),
                ((c.n_heads, c.value_dim, c.key_dim), torch.float32)]


@DSRecurrentMixerRegistry.register_module
class DSGatedDeltaMixer(_RecurrentMixer):
    """Gated delta rule.  Projection columns: ``q (G n) | k (G n) | v (H dv) | gate (H dv) | b (H) | a (H)``; q, k, v pass
    a short convolution + SiLU, q and k become unit vectors (q also times ``n^-1/2``), ``beta = sigmoid(b)``,
    ``decay = exp(-exp(A_log) softplus(a + dt_bias))``; per head ``S <- decay S; S <- S + k (beta (v - S^T k))^T;
    o = S^T q``; the output is ``rms_norm(o) * norm * silu(gate)`` per head."""

    @staticmethod
    def name() -> str:
        return "gated_delta_mixer"

    @staticmethod
    def supports_config(config: DSRecurrentMixerConfig) -> bool:
        return (config.kind == "delta" and config.key_dim <= 256 and 1 <= config.conv_taps <= 16
                and config.n_heads % config.n_heads_kv == 0)

    @property
    def conv_channels(self) -> int:
        c = self._config
        return 2 * c.n_heads_kv * c.key_dim + c.n_heads * c.value_dim

    @property
    def projection_width(self) -> int:
        c = self._config
        return self.conv_channels + c.n_heads * c.value_dim + 2 * c.n_heads

    def forward(self, projected, weights, states, batch):
        c = self._config
        H, G, n, dv = c.n_heads, c.n_heads_kv, c.key_dim, c.value_dim
        C = self.conv_channels
        conv_state, S = states
        info, t2s = batch.seq_info(), batch.token_to_seq()
        xin = projected[:, :C]
        x = M.conv_silu(xin, weights.conv_w, None, conv_state, info, t2s)
        M.conv_state_update(xin, conv_state, info)
        M.unit_norm_heads(x, 0, G, n, n ** -0.5, c.unit_norm_eps)
        M.unit_norm_heads(x, G * n, G, n, 1.0, c.unit_norm_eps)
        g0 = C + H * dv
        decay, beta = M.recurrence_gates(projected[:, g0 + H: g0 + 2 * H], projected[:, g0: g0 + H], weights.A_log,
                                         weights.dt_bias, "delta")
        o = M.linear_recurrence(x[:, G * n: 2 * G * n], x[:, : G * n], x[:, 2 * G * n:], decay, beta, None, S, info, H, G,
                                n, dv, True)
        return M.group_norm_gate(o, projected[:, C: C + H * dv], weights.norm, dv, c.eps, False,
                                 _dt(c.output_dtype).torch)


@DSRecurrentMixerRegistry.register_module
class DSChannelDeltaMixer(_RecurrentMixer):
    """Gated delta rule whose decay differs per key channel.  Projection columns: ``q (G n) | k (G n) | v (H dv) | b (H,
    padded to a multiple of 8) | a (ra) | g (rg)``; q, k, v pass a short convolution + SiLU, q and k become unit vectors (q also times ``n^-1/2``),
    ``beta = sigmoid(b)``.  The decay comes from a two-step projection: ``decay[h, c] = exp(-exp(A_log[h]) softplus(
    (w_a2 a)[h n + c] + dt_bias[h n + c]))``, one factor per (head, key channel) pair that multiplies the rows of the matrix
    memory belonging to that channel; then ``u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.  The output is ``o /
    rms(o) * norm * sigmoid(w_g2 g)`` per head.  ``weights``: ``conv_w`` ``[2 G n + H dv, taps]``, ``A_log`` fp32 ``[H]``,
    ``dt_bias`` fp32 ``[H n]``, ``w_a2`` ``[H n, ra]``, ``w_g2`` ``[H dv, rg]``, ``norm`` ``[dv]``."""

    @staticmethod
    def name() -> str:
        return "channel_delta_mixer"

    @staticmethod
    def supports_config(config: DSRecurrentMixerConfig) -> bool:
        return (config.kind == "channel_delta" and config.key_dim <= 256 and 1 <= config.conv_taps <= 16
                and config.n_heads % config.n_heads_kv == 0)

    @property
    def conv_channels(self) -> int:
        c = self._config
        return 2 * c.n_heads_kv * c.key_dim + c.n_heads * c.value_dim

    def forward(self, projected, weights, states, batch):
        c = self._config
        H, G, n, dv = c.n_heads, c.n_heads_kv, c.key_dim, c.value_dim
        C = self.conv_channels
        conv_state, S = states
        info, t2s = batch.seq_info(), batch.token_to_seq()
        xin = projected[:, :C]
        x = M.conv_silu(xin, weights.conv_w, None, conv_state, info, t2s)
        M.conv_state_update(xin, conv_state, info)
        M.unit_norm_heads(x, 0, G, n, n ** -0.5, c.unit_norm_eps)
        M.unit_norm_heads(x, G * n, G, n, 1.0, c.unit_norm_eps)
        ra, rg = weights.w_a2.shape[1], weights.w_g2.shape[1]
        a0 = C + (H + 7) // 8 * 8
        a_raw = F.linear(projected[:, a0: a0 + ra], weights.w_a2)[:, : H * n]
        gate = F.linear(projected[:, a0 + ra: a0 + ra + rg], weights.w_g2)[:, : H * dv]
        decay, beta = M.channel_decay_gates(a_raw, projected[:, C: C + H], weights.A_log, weights.dt_bias, H, n)
        o = M.linear_recurrence(x[:, G * n: 2 * G * n], x[:, : G * n], x[:, 2 * G * n:], decay, beta, None, S, info, H, G,
                                n, dv, True)
        return M.group_norm_gate(o, gate, weights.norm, dv, c.eps, False, _dt(c.output_dtype).torch, sigmoid=True)


@DSRecurrentMixerRegistry.register_module
class DSStateSpaceDualMixer(_RecurrentMixer):
    """State-space duality.  Projection columns: ``z (H dv) | x (H dv) | B (G n) | C (G n) | dt (H)``; x | B | C pass one
    short convolution (with bias) + SiLU; ``dt = softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S +
    dt B x^T; y = S^T C + D x``; the output is ``rms_norm(y * silu(z))`` over ``norm_groups`` equal parts times ``norm``."""

    @staticmethod
    def name() -> str:
        return "ssd_mixer"

    @staticmethod
    def supports_config(config: DSRecurrentMixerConfig) -> bool:
        inner = config.n_heads * config.value_dim
        return (config.kind == "ssd" and config.key_dim <= 256 and 1 <= config.conv_taps <= 16
                and config.n_heads % config.n_heads_kv == 0 and inner % config.norm_groups == 0)

    @property
    def conv_channels(self) -> int:
        c = self._config
        return c.n_heads * c.value_dim + 2 * c.n_heads_kv * c.key_dim

    @property
    def projection_width(self) -> int:
        c = self._config
        return c.n_heads * c.value_dim + self.conv_channels + c.n_heads

    def forward(self, projected, weights, states, batch):
        c = self._config
        H, G, n, dv = c.n_heads, c.n_heads_kv, c.key_dim, c.value_dim
        inner, C = H * dv, self.conv_channels
        conv_state, S = states
        info, t2s = batch.seq_info(), batch.token_to_seq()
        xin = projected[:, inner: inner + C]
        x = M.conv_silu(xin, weights.conv_w, weights.conv_b, conv_state, info, t2s)
        M.conv_state_update(xin, conv_state, info)
        decay, dt = M.recurrence_gates(projected[:, inner + C: inner + C + H], None, weights.A_log, weights.dt_bias,
                                       "ssd")
        y = M.linear_recurrence(x[:, inner: inner + G * n], x[:, inner + G * n:], x[:, :inner], decay, dt, weights.D, S,
                                info, H, G, n, dv, False)
        return M.group_norm_gate(y, projected[:, :inner], weights.norm, inner // c.norm_groups, c.eps, True,
                                 _dt(c.output_dtype).torch)


@DSRecurrentMixerRegistry.register_module
class DSMatrixLSTMMixer(_RecurrentMixer):
    """Matrix-memory LSTM.  Projection columns: ``q (H n) | k (H n) | v (H dv) | gate (H dv) | i (H) | f (H)``.  Log gates
    ``i = cap tanh((i + b_i) / cap)``, ``f = logsigmoid(cap tanh((f + b_f) / cap))``; with a running maximum ``m`` (0 at
    the start) ``m_t = max(f + m, i)``, ``S <- exp(f + m - m_t) S + exp(i - m_t) k v^T``, ``z`` likewise with ``k`` alone,
    ``o = S^T q / (max(|z . q|, exp(-m_t)) + 1e-6)`` with ``q`` scaled by ``n^-1/2``; the output is ``o / rms(o)`` per
    head times ``norm`` times ``sigmoid(gate)``.  ``z`` is carried as one more value channel that is always 1, so the
    state per head is ``[dv + 1, n]`` and the recurrence the same kernel the other mixers use."""

    @staticmethod
    def name() -> str:
        return "mlstm_mixer"

    @staticmethod
    def supports_config(config: DSRecurrentMixerConfig) -> bool:
        return (config.kind == "mlstm" and config.key_dim <= 256 and config.n_heads == config.n_heads_kv
                and config.gate_cap > 0.0)

    @property
    def conv_channels(self) -> int:
        return 0

    @property
    def projection_width(self) -> int:
        c = self._config
        return 2 * c.n_heads * (c.key_dim + c.value_dim) + 2 * c.n_heads

    def state_shapes(self):
        """Matrix state with the normaliser as its last row per head, and the running maximum."""
        c = self._config
        return [((c.n_heads, c.value_dim + 1, c.key_dim), torch.float32), ((c.n_heads,), torch.float32)]

    def forward(self, projected, weights, states, batch):
        c = self._config
        H, n, dv = c.n_heads, c.key_dim, c.value_dim
        S, m = states
        info = batch.seq_info()
        g0 = 2 * H * n + H * dv
        i0 = g0 + H * dv
        decay, beta, mt = M.mlstm_gate_scan(projected[:, i0: i0 + H], projected[:, i0 + H: i0 + 2 * H], weights.gate_bias_i,
                                            weights.gate_bias_f, c.gate_cap, m, info)
        x = M.mlstm_prepare(projected, H, n, dv, n ** -0.5)
        o = M.linear_recurrence(x[:, H * n: 2 * H * n], x[:, : H * n], x[:, 2 * H * n:], decay, beta, None, S, info, H, H,
                                n, dv + 1, False)
        return M.mlstm_output(o, mt, projected[:, g0: g0 + H * dv], weights.norm, H, dv, c.eps,
                              _dt(c.output_dtype).torch)


@DSSelfAttentionRegistry.register_module
class DSLatentSinkAttention(DSSelfAttentionBase):
    """Attention whose keys and values are up-projections of one normalised latent vector per token.  The paged cache
    holds, per token, that latent (``kv_latent_dim`` channels) followed by one rotated key part (``rope_head_dim``
    channels, interleaved pairs) shared by all heads -- nothing per head.  Queries come through a normalised latent of
    their own.  The up-projections never run over the cache: a query head's unrotated part is carried through the key
    up-projection (``q_abs = W_uk[h]^T q``), attention runs in the latent space with ``[q_abs | q_rot]`` against
    ``[latent | k_rot]`` and the latent itself as value, and the value up-projection is applied to the attended latent.
    Causal or sliding-window mask, optional sink logit; scores, weights and the weighted sum are fp32.  With
    ``q_direct`` the queries are columns of the fused projection itself (no query latent).  ``rotary_scaling`` slows
    the long-wavelength pairs of the rotation (see :class:`RotaryScalingConfig`) and scales cos and sin.  With
    ``output_gate`` the heads' outputs are multiplied by the sigmoid of further columns of the fused projection: one
    per output channel, or one per head (``output_gate_per_head``).

    ``forward(projected, cache, batch, inv_freqs, weights)``: ``projected`` ``[T, q_rank + kv_latent_dim +
    rope_head_dim (+ gate columns) (+ padding)]`` is the fused down-projection (``q_direct``: ``H (d + rot)`` query
    columns in place of the ``q_rank`` latent ones); ``weights`` has ``q_norm``, ``w_uq`` ``[H (d + rot), q_rank]`` (not
    with ``q_direct``), ``kv_norm``, ``w_uk`` ``[H, d, r]``, ``w_uv_t`` ``[H, r, dv]`` and ``sink``.  Returns ``[T, H dv]``."""

    @staticmethod
    def name() -> str:
        return "latent_sink_attention"

    @staticmethod
    def supports_config(config: DSSelfAttentionConfig) -> bool:
        if config.kv_latent_dim is None or config.rope_head_dim < 0 or config.n_heads_kv != 1:
            return False
        if MaskingType(config.masking_type) not in (MaskingType.causal, MaskingType.sliding_window):
            return False
        if MaskingType(config.masking_type) == MaskingType.sliding_window and int(config.masking_args.get("size", 0)) < 1:
            return False
        return PositionalEmbeddingType(config.positional_embedding_type) in (PositionalEmbeddingType.none,
                                                                             PositionalEmbeddingType.rotate_every_other)

    def __init__(self, config: DSSelfAttentionConfig, implementation_config: Dict[str, Any]) -> None:
        super().__init__(config, implementation_config)
        rot = config.positional_embedding_config
        n_rot = 0
        if PositionalEmbeddingType(config.positional_embedding_type) == PositionalEmbeddingType.rotate_every_other:
            n_rot = config.rope_head_dim if rot is None or rot.rotate_dim is None else rot.rotate_dim
        if n_rot % 2 or n_rot > config.rope_head_dim:
            raise ValueError(f"cannot rotate {n_rot} of {config.rope_head_dim} channels in pairs")
        base = 10000.0 if rot is None else rot.theta_base
        self._inv_freq, self._rot_amp = self.rotary_table(n_rot, base, config.rotary_scaling)

    @staticmethod
    def rotary_table(n_rot: int, base: float, scaling=None):
        """fp32 angular frequencies ``base^(-2i / n_rot)`` of the ``n_rot / 2`` pairs and the factor on cos and sin.  With
        ``scaling``: let ``pair(t) = n_rot ln(original / (2 pi t)) / (2 ln base)`` be the (fractional) pair that makes
        ``t`` turns over the original context, ``lo = max(floor(pair(fast)), 0)``, ``hi = min(ceil(pair(slow)), n_rot - 1)``
        and ``w_i = min(1, max(0, (i - lo) / max(hi - lo, 0.001)))``; pair ``i`` turns at ``f_i (1 - w_i) + w_i f_i /
        factor`` and the amplitude is ``0.1 ln(factor) + 1``.  Evaluated in float64, stored as float32."""
        i = torch.arange(0, n_rot, 2, dtype=torch.float64) / 2.0
        f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / max(n_rot, 1))
        amp = 1.0
        if scaling is not None and n_rot > 0:
            def pair(turns: float) -> float:
                return n_rot * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            lo = max(math.floor(pair(scaling.fast)), 0)
            hi = min(math.ceil(pair(scaling.slow)), n_rot - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / scaling.factor * ramp + f * (1.0 - ramp)
            amp = 0.1 * math.log(scaling.factor) + 1.0
        return f.to(torch.float32), float(amp)

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    @property
    def cache_row(self) -> int:
        return self._config.kv_latent_dim + self._config.rope_head_dim

    MAX_VALUE_COLS = 256        # the attention kernels hold at most this many value channels per query head

    def forward(self, projected: torch.Tensor, kv_cache, batch, inv_freqs=None, weights=None) -> torch.Tensor:
        c = self._config
        H, d, rot, r, dv = c.n_heads_q, c.head_size, c.rope_head_dim, c.kv_latent_dim, c.v_head_size or c.head_size
        cache = kv_cache[0] if isinstance(kv_cache, (tuple, list)) else kv_cache
        T = projected.shape[0]
        if self._inv_freq.device != projected.device:
            self._inv_freq = self._inv_freq.to(projected.device)
        t2s, pos, tables = batch.token_to_seq(), batch.token_positions(), batch.block_tables()
        if c.q_direct:
            q_rank = H * (d + rot)
            q = projected[:, :q_rank]                                          # [T, H (d + rot)], a column slice
            q_nope = q.unflatten(1, (H, d + rot))[:, :, :d].transpose(0, 1)    # [H, T, d], strided
        else:
            q_rank = weights.w_uq.shape[1]
            cq = M.rms_norm_slice(projected[:, :q_rank], weights.q_norm, c.qk_norm_eps)
            q = F.linear(cq, weights.w_uq)[:, : H * (d + rot)]                 # [T, H (d + rot)]
            q_nope = q.unflatten(1, (H, d + rot))[:, :, :d].transpose(0, 1)    # [H, T, d]
        q_abs = torch.bmm(q_nope, weights.w_uk).transpose(0, 1)               # [T, H, r], strided
        qf = M.latent_qk_prepare(q, q_abs, projected[:, q_rank: q_rank + r + rot], weights.kv_norm, self._inv_freq, cache,
                                 t2s, pos, tables, H, d, rot, c.qk_norm_eps, self._rot_amp)
        window = int(c.masking_args["size"]) if MaskingType(c.masking_type) == MaskingType.sliding_window else 0
        out_dt = _dt(c.output_dtype).torch
        atoms, n_long = None, 0
        if qf.is_cuda and hasattr(batch, "atoms_longer_than"):
            atoms, n_long = batch.atoms(), batch.atoms_longer_than(M.SHORT_ATOM)
        sink = weights.sink if c.sink else None
        if r <= self.MAX_VALUE_COLS:
            lat = M.sink_attention(qf, cache, None, sink, t2s, pos, tables, c.scale_factor, 0, out_dt, atoms, n_long,
                                   window=window, value_cols=r)
        else:
            # wider latents: the value channels in parts, each a pass over the keys with the same weights
            parts = []
            for c0 in range(0, r, self.MAX_VALUE_COLS):
                n = min(self.MAX_VALUE_COLS, r - c0)
                parts.append(M.sink_attention(qf, cache, None, sink, t2s, pos, tables, c.scale_factor, 0, out_dt, None, 0,
                                              window=window, value_cols=n, value_col0=c0).view(T, H, n))
            lat = torch.cat(parts, dim=2)
        ctx = torch.bmm(lat.view(T, H, r).transpose(0, 1), weights.w_uv_t)     # [H, T, dv]
        ctx = ctx.transpose(0, 1).reshape(T, H * dv)
        if c.output_gate:
            g0 = q_rank + r + rot
            if c.output_gate_per_head:
                M.sigmoid_gate_rows_(ctx, projected[:, g0: g0 + H], dv)
            else:
                M.sigmoid_gate_rows_(ctx, projected[:, g0: g0 + H * dv], 1)
        return ctx


@DSPostNormRegistry.register_module
class DSScaledPostRMSNorm(DSPostNormBase):
    """Post-norm on the sublayer's output only, on an fp32 stream: ``x <- x + scale (.) (rms_norm(hidden) * gain)`` with
    ONE gain for all channels and a per-channel ``scale``.  With ``mix`` the result is also stored as the next entry of
    a stack of streams and the stream handed on is their weighted sum (``mix = (stack, n_prev, weights, out)``)."""

    @staticmethod
    def name() -> str:
        return "fp32_scaled_post_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return NormTypeEnum(config.type) == NormTypeEnum.RMSNorm and _dt(config.residual_dtype) == DtypeEnum.fp32

    def forward(self, residual, hidden_states, gamma, beta=None, scale=None, out=None, mix=None):
        out = residual if out is None else out
        if mix is None:
            M.post_norm_mix(residual, hidden_states, gamma, scale, out, self._config.eps)
        else:
            stack, n_prev, w, mixed = mix
            M.post_norm_mix(residual, hidden_states, gamma, scale, out, self._config.eps, stack, n_prev, w, mixed)
        return out


@DSSelfAttentionRegistry.register_module
class DSFilteredBiasAttention(DSSelfAttentionBase):
    """Softmax attention without rotation whose projections pass a short causal filter over time.  Projection columns:
    ``q (Hq d) | k (G d) | v (G dv) | gate (Hq dv)``.  Every channel of q | k | v is filtered over the sequence (the last
    ``taps - 1`` projected rows are carried per sequence), q and k heads are RMS-normed with one weight of ``d`` entries
    each, q is multiplied by ``1 + coef * ln(floor((pos + 1) / every) + 1)``; a key at distance ``n`` behind the query
    adds the learned ``bias[bucket(n), h]`` to its scaled score (buckets: one per distance below half the table's rows,
    logarithmic up to ``far`` above); causal or chunk-local / sliding-window mask; the heads' outputs are multiplied by
    ``sigmoid(gate)``.  Filter sums, norms, temperature, scores, weights and the weighted sum are fp32; the paged cache
    holds the normalised keys and the filtered values in the activation dtype.

    ``forward(projected, (keys, values), batch, inv_freqs, weights, conv_state)``: ``weights`` has ``conv_w`` ``[C,
    taps]`` (or None), ``q_norm`` / ``k_norm`` (or None) and ``dist_bias`` (fp32 ``[Hq, distances]`` from
    :meth:`expand_distance_bias`, or None)."""

    @staticmethod
    def name() -> str:
        return "filtered_bias_attention"

    @staticmethod
    def supports_config(config: DSSelfAttentionConfig) -> bool:
        if config.kv_latent_dim is not None or config.sink:
            return False
        if MaskingType(config.masking_type) not in (MaskingType.causal, MaskingType.chunked, MaskingType.sliding_window):
            return False
        pe = PositionalEmbeddingType(config.positional_embedding_type)
        if pe == PositionalEmbeddingType.distance_bias:
            b = config.distance_bias
            if b is None or b.rows < 2 or b.far <= b.rows // 2:
                return False
        elif pe != PositionalEmbeddingType.none:
            return False
        return (config.head_size <= 256 and (config.v_head_size or config.head_size) <= 256
                and config.n_heads_q % config.n_heads_kv == 0 and 1 <= config.qkv_conv_taps <= 16
                and config.q_temp_every >= 1)

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    @property
    def filtered_channels(self) -> int:
        c = self._config
        return (c.n_heads_q + c.n_heads_kv) * c.head_size + c.n_heads_kv * (c.v_head_size or c.head_size)

    @property
    def projection_width(self) -> int:
        c = self._config
        return self.filtered_channels + (c.n_heads_q * (c.v_head_size or c.head_size) if c.output_gate else 0)

    def state_shapes(self):
        """[(shape per sequence, dtype)]: the filter's carried inputs (none for a single tap)."""
        c = self._config
        if c.qkv_conv_taps <= 1:
            return []
        return [((c.qkv_conv_taps - 1, self.filtered_channels), _dt(c.input_dtype).torch)]

    @staticmethod
    def bucket_of_distance(rows: int, far: int) -> torch.Tensor:
        """int64 ``[far + 1]``: the table row of every distance ``0 .. far``; larger distances use the last entry (the
        last row).  ``bucket(n) = n`` below ``half = rows // 2``, else ``min(rows - 1, half + floor(ln(n / half) /
        ln(far / half) * (rows - half)))``."""
        half = rows // 2
        n = torch.arange(far + 1, dtype=torch.float64)
        ratio = torch.log(n.clamp(min=1) / max(half, 1)) / math.log(far / max(half, 1)) * (rows - half)
        large = (half + torch.floor(ratio + 1e-9).long()).clamp(max=rows - 1)
        return torch.where(n < half, n.long(), large)

    @staticmethod
    def expand_distance_bias(table: torch.Tensor, far: int) -> torch.Tensor:
        """A checkpoint's ``[rows, Hq]`` table as fp32 ``[Hq, far + 1]`` indexed by the distance itself."""
        idx = DSFilteredBiasAttention.bucket_of_distance(table.shape[0], far).to(table.device)
        return table.float().index_select(0, idx).t().contiguous()

    def forward(self, projected: torch.Tensor, kv_cache, batch, inv_freqs=None, weights=None,
                conv_state=None) -> torch.Tensor:
        c = self._config
        dv = c.v_head_size or c.head_size
        keys, values = kv_cache
        C = self.filtered_channels
        t2s, pos, tables, info = batch.token_to_seq(), batch.token_positions(), batch.block_tables(), batch.seq_info()
        conv_w = getattr(weights, "conv_w", None)          # one tap: a scale per channel, nothing carried
        q = M.qkv_filter_norm_append(projected, conv_w, conv_state, info, weights.q_norm if c.qk_norm_weight else None,
                                     weights.k_norm if c.qk_norm_weight else None, keys, values, t2s, pos, tables,
                                     c.n_heads_q, c.n_heads_kv, c.head_size, dv, c.qk_norm_eps, True, c.q_temp_coef,
                                     c.q_temp_every)
        if conv_w is not None and conv_w.shape[1] > 1:
            M.conv_state_update(projected[:, :C], conv_state, info)
        mt = MaskingType(c.masking_type)
        chunk = int(c.masking_args["size"]) if mt == MaskingType.chunked else 0
        window = int(c.masking_args["size"]) if mt == MaskingType.sliding_window else 0
        atoms, n_long = None, 0
        if q.is_cuda and M.tiles_supported(c.head_size, dv) and hasattr(batch, "atoms_longer_than"):
            atoms, n_long = batch.atoms(), batch.atoms_longer_than(M.SHORT_ATOM)
        bias = weights.dist_bias if c.distance_bias is not None else None
        gate = projected[:, C: C + c.n_heads_q * dv] if c.output_gate else None
        return M.sink_attention(q, keys, values, None, t2s, pos, tables, c.scale_factor, chunk, _dt(c.output_dtype).torch,
                                atoms, n_long, window=window, dist_bias=bias, gate=gate)
