"""Module configs (reference ``inference/v2/modules/configs/*``)."""
from enum import Enum
from typing import Dict, Optional

from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum
from ..ds_module import DSModuleConfig
from .....runtime.config_utils import DeepSpeedConfigModel


class PositionalEmbeddingType(Enum):
    none = "none"
    rotate_half = "rotate_half"
    rotate_every_other = "rotate_every_other"
    alibi = "alibi"
    distance_bias = "distance_bias"    # a learned bias per head and bucket of the distance query - key, added to the score


class DistanceBiasConfig(DeepSpeedConfigModel):
    """Buckets of a learned distance bias: a table with ``rows`` rows per head; distances below ``rows // 2`` have a row
    each, the others share rows on a logarithmic scale that reaches the last row at ``far``."""
    rows: int
    far: int


class RotateHalfConfig(DeepSpeedConfigModel):
    use_trained_freqs: bool = False
    theta_base: float = 10_000.0
    rotate_dim: Optional[int] = None      # None: rotate the whole head; < head_size: partial rotary (Phi, GPT-NeoX)


class RotaryScalingConfig(DeepSpeedConfigModel):
    """Frequency interpolation by wavelength for contexts ``factor`` times longer than ``original`` positions: pairs
    that complete fewer than ``slow`` turns over the original context are slowed by ``factor``, pairs with more than
    ``fast`` turns keep their frequency, the ones between are blended along a linear ramp over the pair index; cos and
    sin carry the factor ``1 + 0.1 ln(factor)``."""
    factor: float
    original: float
    fast: float = 32.0
    slow: float = 1.0


class MaskingType(Enum):
    none = "none"
    causal = "causal"
    local = "local"
    symmetric = "symmetric"
    asymmetric = "asymmetric"
    chunked = "chunked"      # causal inside aligned chunks of ``masking_args["size"]`` positions, nothing across chunks
    sliding_window = "sliding_window"   # causal over the query and the ``masking_args["size"] - 1`` positions before it


class DSSelfAttentionConfig(DSModuleConfig):
    n_heads_q: int
    n_heads_kv: int
    head_size: int
    max_sequences: int
    scale_factor: float = 1.0
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16
    masking_type: MaskingType = MaskingType.causal
    masking_args: Dict = {}
    positional_embedding_type: PositionalEmbeddingType = PositionalEmbeddingType.none
    positional_embedding_config: Optional[RotateHalfConfig] = None
    v_head_size: Optional[int] = None     # value head size when it differs from the query / key head size
    qk_unit_rms: bool = False             # divide every query / key head by its root mean square (no weight)
    qk_norm_eps: float = 1e-5
    sink: bool = False                    # one learned logit per head joins the softmax denominator
    # Latent attention: keys and values are up-projections of one normalised latent vector of ``kv_latent_dim`` channels
    # per token, and every query / key head has ``rope_head_dim`` further channels that carry the rotation (the key's are
    # shared by all heads).  ``head_size`` is then the unrotated query / key head size and the cache holds
    # ``kv_latent_dim + rope_head_dim`` channels per token.
    kv_latent_dim: Optional[int] = None
    rope_head_dim: int = 0
    # Projections that pass a short causal filter over time (``qkv_conv_taps`` taps per channel of q | k | v; the last
    # ``taps - 1`` projected rows of a sequence are carried state) before the per-head norm.
    qkv_conv_taps: int = 1
    qk_norm_weight: bool = False          # the per-head RMS norm of q and k has a weight of head_size entries each
    # Query temperature: q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
    q_temp_coef: float = 0.0
    q_temp_every: int = 1
    distance_bias: Optional[DistanceBiasConfig] = None      # with PositionalEmbeddingType.distance_bias
    output_gate: bool = False             # the heads' outputs are multiplied by sigmoid of one more projection
    output_gate_per_head: bool = False    # that projection has one output per head instead of one per output channel
    # Latent attention: the queries are projected straight from the input (``H (head_size + rope_head_dim)`` columns
    # at the start of the fused projection) instead of through a normalised latent with an up-projection.
    q_direct: bool = False
    rotary_scaling: Optional[RotaryScalingConfig] = None


class DSEmbeddingsConfig(DSModuleConfig):
    residual_dtype: DtypeEnum = DtypeEnum.bf16
    embedding_dim: int
    positional_embedding: bool = False
    positional_offset: int = 0            # OPT stores position p at row p + 2
    use_token_type: bool = False
    output_normalization: Optional[NormTypeEnum] = None
    scale: float = 1.0                    # multiplies the token rows
    sinusoid_base: Optional[float] = None  # adds interleaved sin / cos of pos * base^(-2i/dim) when set
    widen_to_residual: bool = False       # the stream is fp32 whatever the table's dtype: rows are converted on the way


class DSLinearConfig(DSModuleConfig):
    in_channels: int
    out_channels: int                     # after gating: a gated layer's weight is [2 * out_channels, in_channels]
    activation: ActivationType = ActivationType.IDENTITY
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16


class DSMoEConfig(DSModuleConfig):
    model_dim: int
    intermediate_features: int
    n_experts: int
    top_k: int = 1
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16
    activation: ActivationType = ActivationType.IDENTITY
    normalize_scores: bool = False
    score_function: str = "softmax"       # "softmax" over all experts, or "sigmoid" of every expert's own logit
    weight_input: bool = False            # the routing weight scales the expert's input instead of its output
    router_dtype: Optional[DtypeEnum] = None    # dtype of the router product (None: the activation dtype)
    router_bias: bool = False             # the router logits have a bias
    # A shared expert of ``shared_features`` channels runs for every token; its output is multiplied by the sigmoid of
    # one more router row (the row after the experts' rows) and added.
    shared_features: int = 0
    # Group-limited choice: the router has ``n_experts + identity_experts`` outputs in ``n_groups`` equal groups of
    # neighbours; the winners are the ``top_k`` largest ``score + correction`` inside the ``keep_groups`` groups whose
    # best member is largest; the weights are the winners' plain scores / their sum * ``score_scale``.  The last
    # ``identity_experts`` outputs stand for experts that return their input (they have no weights).
    score_correction: bool = False
    n_groups: int = 1
    keep_groups: int = 1
    score_scale: float = 1.0
    identity_experts: int = 0
    activation_limit: float = 0.0         # ActivationType.CLAMPED_SWIGLU: the clamp


class DSNormConfig(DSModuleConfig):
    type: NormTypeEnum
    channels: int
    residual_dtype: DtypeEnum = DtypeEnum.bf16
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16
    eps: float = 1e-5


class DSUnembedConfig(DSModuleConfig):
    dtype: DtypeEnum = DtypeEnum.bf16
    norm_type: Optional[NormTypeEnum] = None
    model_dim: int
    max_sequences: int
    vocab_size: int
    eps: float = 1e-5


class DSRecurrentMixerConfig(DSModuleConfig):
    """A token mixer that carries a matrix state per head instead of a key / value cache.

    ``kind`` ``"delta"``: gated delta rule (keys / queries of ``key_dim`` channels shared by ``n_heads // n_heads_kv``
    value heads, short convolutions on q, k, v).  ``"channel_delta"``: the same rule with one decay per head and key
    channel (from a two-step projection), a sigmoid write strength and a sigmoid output gate from a second two-step
    projection behind the per-head norm.  ``"ssd"``: state-space duality (B / C of ``key_dim`` = state size per
    group, a convolution over x | B | C, a skip term and a gated group norm).  ``"mlstm"``: matrix-memory LSTM
    (exponential input gate, sigmoid forget gate in log space, both capped by ``gate_cap``, a running maximum that
    keeps the exponentials in range, a normaliser state, per-head unit-RMS and a sigmoid output gate; no convolution)."""
    kind: str
    model_dim: int
    n_heads: int
    n_heads_kv: int                       # key/query heads (delta) or B/C groups (ssd)
    key_dim: int
    value_dim: int
    conv_taps: int = 1
    norm_groups: int = 1
    gate_cap: float = 0.0                 # mlstm: gate pre-activations pass cap * tanh(x / cap)
    eps: float = 1e-5
    unit_norm_eps: float = 1e-6
    max_sequences: int = 1
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16
