"""Pick a module implementation for a config (reference ``inference/v2/modules/heuristics.py:35-195``)."""
from __future__ import annotations

from ..config_v2 import RaggedInferenceEngineConfig
from ..inference_utils import NormTypeEnum
from . import implementations  # noqa: F401  (registers the implementations)
from .configs import (DSEmbeddingsConfig, DSLinearConfig, DSMoEConfig, DSNormConfig, DSRecurrentMixerConfig,
                      DSSelfAttentionConfig, DSUnembedConfig)
from .interfaces import (DSEmbeddingBase, DSEmbeddingRegistry, DSLinearBase, DSLinearRegistry, DSMoEBase,
                         DSMoERegistry, DSPostNormBase, DSPostNormRegistry, DSPreNormBase, DSPreNormRegistry,
                         DSRecurrentMixerBase, DSRecurrentMixerRegistry, DSSelfAttentionBase, DSSelfAttentionRegistry,
                         DSUnembedBase, DSUnembedRegistry)
from .module_registry import ConfigBundle


def instantiate_attention(attention_config: DSSelfAttentionConfig,
                          engine_config: RaggedInferenceEngineConfig) -> DSSelfAttentionBase:
    if attention_config.kv_latent_dim is not None:
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="latent_sink_attention",
                                                                       config=attention_config))
    name = "dense_blocked_attention"
    if not DSSelfAttentionRegistry.registry[name].supports_config(attention_config):
        name = "sink_chunked_attention"       # chunk-local mask, sink logit, q/k unit norm or narrower value heads
    if not DSSelfAttentionRegistry.registry[name].supports_config(attention_config):
        name = "filtered_bias_attention"      # filtered projections, weighted q/k norm, distance bias, output gate
    return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name=name, config=attention_config))


def instantiate_embed(embed_config: DSEmbeddingsConfig, engine_config: RaggedInferenceEngineConfig) -> DSEmbeddingBase:
    widen = embed_config.widen_to_residual or embed_config.sinusoid_base is not None
    name = "scaled_sinusoid_embedding" if widen else "ragged_embedding"
    return DSEmbeddingRegistry.instantiate_config(ConfigBundle(name=name, config=embed_config))


def instantiate_linear(linear_config: DSLinearConfig, engine_config: RaggedInferenceEngineConfig) -> DSLinearBase:
    mode = getattr(getattr(engine_config, "quantization", None), "quantization_mode", None)
    if mode is None:
        name = "blas_fp_linear"
    elif mode == "wf6af16":
        name = "quantized_wf6af16_linear"
        impl = DSLinearRegistry.registry[name]
        if not impl.supports_config(linear_config):
            name = "blas_fp_linear"       # shapes the FP6 layout cannot hold stay in 16-bit
    else:
        raise ValueError(f"Unsupported quantization mode: {mode}")
    return DSLinearRegistry.instantiate_config(ConfigBundle(name=name, config=linear_config))


def instantiate_moe(moe_config: DSMoEConfig, engine_config: RaggedInferenceEngineConfig) -> DSMoEBase:
    return DSMoERegistry.instantiate_config(ConfigBundle(name="cutlass_multi_gemm_moe", config=moe_config,
                                                         implementation_config={"weight_dtype": moe_config.input_dtype}))


def instantiate_post_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig) -> DSPostNormBase:
    return DSPostNormRegistry.instantiate_config(ConfigBundle(name="cuda_post_ln", config=norm_config))


def instantiate_pre_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig) -> DSPreNormBase:
    name = "cuda_pre_rms" if NormTypeEnum(norm_config.type) == NormTypeEnum.RMSNorm else "cuda_pre_ln"
    return DSPreNormRegistry.instantiate_config(ConfigBundle(name=name, config=norm_config))


def instantiate_unembed(unembed_config: DSUnembedConfig, engine_config: RaggedInferenceEngineConfig) -> DSUnembedBase:
    return DSUnembedRegistry.instantiate_config(ConfigBundle(name="ragged_unembed", config=unembed_config))


def instantiate_recurrent_mixer(mixer_config: DSRecurrentMixerConfig,
                                engine_config: RaggedInferenceEngineConfig) -> DSRecurrentMixerBase:
    name = {"delta": "gated_delta_mixer", "ssd": "ssd_mixer", "mlstm": "mlstm_mixer",
            "channel_delta": "channel_delta_mixer"}.get(mixer_config.kind)
    if name is None:
        raise ValueError(f"Unknown recurrent mixer kind {mixer_config.kind!r}; expected 'delta', 'channel_delta', 'ssd' "
                         "or 'mlstm'")
    return DSRecurrentMixerRegistry.instantiate_config(ConfigBundle(name=name, config=mixer_config))


def instantiate_sandwich_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig) -> DSPreNormBase:
    """Pre- and post-norm around every sublayer on an fp32 residual stream."""
    return DSPreNormRegistry.instantiate_config(ConfigBundle(name="fp32_sandwich_rms", config=norm_config))


def instantiate_scaled_post_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig) -> DSPostNormBase:
    """Post-norm with one gain and a per-channel scale on an fp32 stream, optionally mixing the streams of all layers."""
    return DSPostNormRegistry.instantiate_config(ConfigBundle(name="fp32_scaled_post_rms", config=norm_config))
