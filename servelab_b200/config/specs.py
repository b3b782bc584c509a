"""Architecture-neutral description of a model as data.

A model is a list of *layers*, each a block that names its parts (mixer,
feed-forward, norms) by registry kind together with their sizes and constants,
plus a *run order*: the sequence in which layers execute, which may name a layer
twice or let a run read the cache that an earlier run filled.  Nothing in here knows any
model family; the family's config class (for example ``Qwen2Config``) translates
its own ``config.json`` keys into these specs.

The specs are frozen dataclasses so they can be hashed, compared and printed.
A spec's ``kind`` selects the implementation from the part registries in
``servelab_b200.parts.registry``; new kinds are added by registering a part
there, never by editing this file.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description: ``kind`` is the registry key."""
    kind: str


# ----------------------------------------------------------------- positions
@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding over the first ``rotary_dim``
    elements of each head (``rotary_dim == head_dim`` for a full rotation)."""
    kind: str = "rotary"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    # Stretching of the long wavelengths (None: none): with wavelength l = 2 pi / f, a frequency
    # with l > stretch_original / stretch_low is divided by ``stretch_factor``, one with
    # l < stretch_original / stretch_high is kept, and between the two
    # s = (stretch_original / l - stretch_low) / (stretch_high - stretch_low) blends them,
    # (1 - s) f / factor + s f.
    stretch_factor: Optional[float] = None
    stretch_low: float = 1.0
    stretch_high: float = 4.0
    stretch_original: float = 8192.0
    precise: bool = False      # the frequencies are formed in float64 and rounded to float32 once


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: str = "none"


@dataclass(frozen=True)
class PairRotarySpec(PartSpec):
    """Rotary encoding that pairs NEIGHBOURING elements (2i with 2i + 1) of ``dims`` elements of
    a head, frequencies f_i = theta^(-2i / dims).  With ``yarn_factor`` the frequencies are
    interpolated between f_i and f_i / factor by a ramp over i that runs from the pair that
    turns ``yarn_fast`` times within ``yarn_original`` positions to the one that turns
    ``yarn_slow`` times, and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    kind: str = "rotary_pairs"
    dims: int = 0
    theta: float = 10000.0
    yarn_factor: Optional[float] = None
    yarn_original: float = 0.0
    yarn_fast: float = 32.0
    yarn_slow: float = 1.0
    # stretching of the long wavelengths as ``RotarySpec`` describes it (None: none)
    stretch_factor: Optional[float] = None
    stretch_low: float = 1.0
    stretch_high: float = 4.0
    stretch_original: float = 8192.0


# --------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    kind: str = "rmsnorm"
    dim: int = 0
    eps: float = 1e-6
    weight_suffix: str = ".weight"         # the weight is <prefix><weight_suffix>
    unit_offset: bool = False              # the stored weight lies around zero: the factor is 1 + w


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """(x - mean) / sqrt(var + eps) * w + b over a row; tensors ``<prefix><weight_suffix>`` and
    ``<prefix><bias_suffix>``."""
    kind: str = "layernorm"
    dim: int = 0
    eps: float = 1e-5
    weight_suffix: str = ".weight"
    bias_suffix: str = ".bias"


@dataclass(frozen=True)
class DynamicTanhSpec(PartSpec):
    """Dynamic Tanh: y = tanh(alpha * x) * w + b per element, with a learned scalar
    ``alpha``; no mean, variance or root mean square is computed.  The three tensors are
    named ``<prefix><weight_suffix>``, ``<prefix><bias_suffix>`` and ``<prefix><alpha_suffix>``."""
    kind: str = "dynamic_tanh"
    dim: int = 0
    weight_suffix: str = ".weight"
    bias_suffix: str = ".bias"
    alpha_suffix: str = ".alpha"


# -------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` is None for attention over all earlier keys, else the number of
    most recent keys (the query's own included) a query may see.
    """
    kind: str = "paged_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None => head_dim ** -0.5
    position: PartSpec = field(default_factory=NoPositionSpec)
    # checkpoint names of the projections under the mixer's prefix (data, like the sizes:
    # an architecture with the same arithmetic and other names changes these, not the part)
    q_name: str = "q_proj"
    k_name: str = "k_proj"
    v_name: str = "v_proj"
    o_name: str = "o_proj"
    position_name: str = "rotary_emb"


@dataclass(frozen=True)
class ConvTalkAttentionSpec(PartSpec):
    """Windowed grouped-query softmax attention whose positions enter through the scores
    alone, with these steps, each a parameter of its own:

    ``conv_taps``        a causal convolution over time on every channel of the projected
                         queries and keys (0: none; 1: a learned factor per channel and no
                         state); the last ``conv_taps - 1`` projected rows of a request are
                         per-request state;
    ``tied_values``      the values are the keys as they leave the convolution (no value
                         projection, keys stored once);
    ``q_temp_coef/every`` queries at position p are multiplied by
                         1 + coef * ln(floor((p + 1) / every) + 1) (coef None: not applied);
    ``distance_bias``    r1_h * ln(1 + r2_h * (i - j)) is subtracted from the scaled score of
                         query i and key j, with two learned numbers a head;
    ``talking_heads``    after the softmax the heads' weights are mixed by a learned [H, H]
                         matrix; head h applies its mixed weights to its own key/value head;
    ``output_gate``      the concatenated heads are multiplied by sigmoid(W_g x) of the
                         mixer's input before the output projection.
    """
    kind: str = "conv_talk_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    scale: Optional[float] = None          # None => head_dim ** -0.5
    conv_taps: int = 0
    tied_values: bool = True
    q_temp_coef: Optional[float] = None
    q_temp_every: int = 1
    distance_bias: bool = False
    talking_heads: bool = False
    output_gate: bool = False
    # checkpoint names under the mixer's prefix
    q_name: str = "q"
    k_name: str = "k"
    o_name: str = "o"
    gate_name: str = "g"
    conv_suffix: str = ".conv"             # the taps of a projection: <projection><conv_suffix>
    bias_r1_name: str = "r1"
    bias_r2_name: str = "r2"
    talk_name: str = "talk"
    weight_suffix: str = ""


@dataclass(frozen=True)
class NormedAttentionSpec(PartSpec):
    """Grouped-query softmax attention whose keys and values may differ in size, with these
    steps, each a parameter:

    ``conv_taps``    a causal convolution over time on every channel of the projected queries,
                     keys and values, directly after the projection (0: none); the last
                     ``conv_taps - 1`` projected rows of a request are per-request state;
    ``qk_norm``      RMS norm over every query and key head before the rotation, one weight
                     vector per projection shared by the heads (``qk_norm_eps``);
    ``position``     a ``PairRotarySpec`` (neighbouring pairs) or a ``RotarySpec`` (element i with
                     element i + dims / 2) on the first ``dims`` elements of a head, or none;
    ``qk_unit_norm`` after the rotation every query and key head is divided by its root mean
                     square (``qk_norm_eps``, no weight);
    ``softcap``      a scaled score s becomes cap tanh(s / cap) (None: not applied);
    ``sink``         one learned number a head whose exponential joins the softmax's denominator
                     (it has no key and no value, is neither scaled nor capped);
    ``value_mix``    None; "source": this layer's values (before any mixing) are kept for the
                     step; "mix": v <- (1 - lambda) v + lambda v_source with a learned scalar,
                     the mixed values being what the cache holds.  ``value_mix_key`` names the
                     source among the layers of a model;
    ``head_gate``    head h's result is multiplied by sigmoid((W_g x)_h), one number a head;
    ``window``       None: every earlier key; else the last ``window`` keys (own included).
    """
    kind: str = "normed_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0                      # queries and keys
    value_dim: int = 0
    window: Optional[int] = None
    scale: Optional[float] = None          # None => head_dim ** -0.5
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    position: PartSpec = field(default_factory=NoPositionSpec)
    value_mix: Optional[str] = None
    value_mix_key: str = "v_first"
    head_gate: bool = False
    conv_taps: int = 0
    qk_unit_norm: bool = False
    softcap: Optional[float] = None
    sink: bool = False
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    gate_name: str = "g"
    q_norm_name: str = "q.norm"
    k_norm_name: str = "k.norm"
    value_mix_name: str = "vmix"
    conv_suffix: str = ".conv"             # the taps of a projection: <projection><conv_suffix>
    sink_name: str = "sink"


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Attention whose keys and values are expanded from one latent vector per token: the
    product W_dkv x gives ``kv_rank`` latent elements (RMS-normed, ``latent_norm_eps``) and
    ``rope_dim`` elements of a rotated key part that all heads share; head h's unrotated key is
    W_uk[h] c and its value W_uv[h] c.  A query head is [``head_dim`` unrotated | ``rope_dim``
    rotated].  Only the latent and the rotated part are cached.  ``element_gate``: the
    concatenated heads are multiplied by sigmoid(W_g x); ``head_gate``: head h's result by
    sigmoid((W_g x)_h), one number a head.  ``q_rank``: the queries come through a latent of
    their own, q = W_uq RMSnorm(W_dq x) (None: q = W_q x).  ``sink``: one learned number a head
    whose exponential joins the softmax's denominator."""
    kind: str = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0                      # unrotated part of queries and keys
    rope_dim: int = 0
    value_dim: int = 0
    kv_rank: int = 0
    window: Optional[int] = None
    scale: Optional[float] = None          # None => (head_dim + rope_dim) ** -0.5
    latent_norm_eps: float = 1e-6
    position: PartSpec = field(default_factory=NoPositionSpec)
    element_gate: bool = False
    head_gate: bool = False
    q_rank: Optional[int] = None
    sink: bool = False
    q_down_name: str = "dq"
    q_norm_name: str = "dq.norm"
    q_up_name: str = "uq"
    sink_name: str = "sink"
    q_name: str = "q"
    down_name: str = "dkv"
    latent_norm_name: str = "dkv.norm"
    up_k_name: str = "uk"
    up_v_name: str = "uv"
    o_name: str = "o"
    gate_name: str = "g"


@dataclass(frozen=True)
class DecayAttentionSpec(PartSpec):
    """Linear attention with a fixed decay per head and a per-request state instead of cached
    keys: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t (no softmax, no denominator), S of
    ``head_dim`` x ``value_dim`` float32 per head.  Around the recurrence, each a parameter:

    ``qkv_activation``  None, or "silu" on the projected q, k and v;
    ``position``        a ``RotarySpec`` (rotate-half over the first ``rotary_dim`` elements of every
                        query and key head) or none;
    ``key_scale``       a factor on the keys (after the rotation); None: 1;
    ``out_norm``        "head": every head's result is divided by its root mean square;
                        "row": the concatenated heads are RMS-normed together;
                        with ``out_norm_weight`` a learned weight over the whole row multiplies;
    ``gate_activation`` the result is multiplied by act(W_g x): "silu" or "sigmoid".

    ``decay_gate_rank``: instead of the fixed ``decay`` (then empty) every key channel of every
    token has a decay of its own, alpha_t = sigmoid(z_t)^(1 / ``decay_gate_tau``) with
    z = W_a2 (W_a1 x) + b through a bottleneck of that many elements, and
    S_t = diag(alpha_t) S_{t-1} + k_t v_t^T.  ``query_scale``: a factor on the queries (None: 1).
    ``out_norm_per_head``: with ``out_norm`` "head" and a weight, the weight has ``value_dim``
    elements and is shared by the heads.
    """
    kind: str = "decay_attention"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    decay: Tuple[float, ...] = ()
    qkv_activation: Optional[str] = None
    position: PartSpec = field(default_factory=NoPositionSpec)
    key_scale: Optional[float] = None
    out_norm: str = "head"
    out_norm_weight: bool = False
    out_norm_eps: float = 1e-6
    gate_activation: str = "silu"
    decay_gate_rank: Optional[int] = None
    decay_gate_tau: float = 1.0
    query_scale: Optional[float] = None
    out_norm_per_head: bool = False
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    out_norm_name: str = "norm"
    decay_down_name: str = "a1"
    decay_up_name: str = "a2"
    decay_bias_name: str = "a2.b"


@dataclass(frozen=True)
class DifferentialAttentionSpec(PartSpec):
    """Grouped-query softmax attention with two maps a head: every query head and every kv head
    carries two query / key vectors of ``head_dim`` elements ([head][map]), each map attends on
    its own over the kv head's one set of values (``value_dim``), and a head's result is
    o = a_1 - lambda a_2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``lambda_init`` (four
    learned vectors of ``head_dim`` elements, one number a layer), divided by its root mean
    square over the head (``norm_eps``, no weight) and multiplied by 1 - ``lambda_init``.  Biases
    on q, k and v; positions do not enter the scores.  ``own_kv`` False: the layer has no key
    and value projections and reads the cache that another layer fills."""
    kind: str = "differential_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    scale: Optional[float] = None          # None => head_dim ** -0.5
    lambda_init: float = 0.0
    norm_eps: float = 1e-6
    qkv_bias: bool = True
    own_kv: bool = True
    window: Optional[int] = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    bias_suffix: str = ".b"
    lambda_names: Tuple[str, str, str, str] = ("lq1", "lk1", "lq2", "lk2")


@dataclass(frozen=True)
class ParallelMixersSpec(PartSpec):
    """Two mixers side by side that read the same input; each one's result is RMS-normed over the
    model width with a weight of its own (``eps``) and the mixer returns ``factor`` times their
    sum.  The branches' tensors live under ``<prefix>.<left_name>`` and ``<prefix>.<right_name>``,
    the norm weights under ``<prefix>.<left_name><out_suffix>`` and the same for the right."""
    kind: str = "parallel_mixers"
    hidden_size: int = 0
    left: PartSpec = None
    right: PartSpec = None
    eps: float = 1e-6
    factor: float = 0.5
    left_name: str = "left"
    right_name: str = "right"
    out_suffix: str = ".out"


# -------------------------------------------------------------- feed-forward
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down(act(gate(x)) * up(x)) with a dense (expert-free) gate/up/down; ``activation``
    "silu", "gelu_tanh" or "swish_clamped": g = min(gate, limit), u = clamp(up, -limit, limit),
    g sigmoid(``swish_alpha`` g) (u + 1)."""
    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    limit: Optional[float] = None          # (swish_clamped)
    swish_alpha: float = 1.702
    bias: bool = False
    gate_name: str = "gate_proj"           # checkpoint names under the feed-forward's prefix
    up_name: str = "up_proj"
    down_name: str = "down_proj"
    weight_suffix: str = ".weight"         # a matrix is <prefix>.<name><weight_suffix>


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """``num_experts`` gated feed-forwards of which a token uses ``top``: scores = softmax of the
    router's float32 logits over all experts; the experts form ``num_groups`` equal groups of
    neighbours, a group scores as its best expert and only the ``keep_groups`` best groups'
    experts can be chosen; the chosen experts' outputs are weighted by their scores times
    ``route_scale`` (divided by the sum of the chosen scores first with ``renormalize``).
    ``shared``: a dense gated feed-forward that every token also passes, added to the sum.
    ``score_fn`` "sigmoid": the scores are sigmoids of the logits.  ``correction_name``: a learned
    offset per expert that is added to the scores for the choice (experts and groups) and not for
    the weights.  ``group_best``: a group scores as the sum of its that many largest choice scores
    (1: its best).  ``norm_eps``: added to the sum of the chosen scores with ``renormalize``."""
    kind: str = "routed_experts"
    hidden_size: int = 0
    num_experts: int = 0
    top: int = 1
    expert_size: int = 0
    num_groups: int = 1
    keep_groups: int = 1
    route_scale: float = 1.0
    renormalize: bool = False
    shared: Optional[PartSpec] = None
    score_fn: str = "softmax"
    correction_name: Optional[str] = None
    group_best: int = 1
    norm_eps: float = 0.0
    router_name: str = "router"
    expert_prefix: str = "e{}"             # expert j's tensors: <prefix>.e<j>.<gate|up|down>
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    shared_name: str = "shared"
    weight_suffix: str = ""


# --------------------------------------------------------------------- block
@dataclass(frozen=True)
class BlockSpec(PartSpec):
    """One layer: how a mixer, a feed-forward and their norms are arranged.
    ``pre_norm`` is x += mixer(norm1(x)); x += ff(norm2(x)).
    ``sandwich_norm`` norms each sublayer's result as well before it is added:
    x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))); its ``feed_forward`` may be
    None (a layer that has a mixer only).
    ``result_norm`` norms only what a sublayer returns; the sublayers read the stream itself:
    x += norm1(mixer(x)); x += norm2(ff(x)) (``mixer_post_norm``, ``ff_post_norm``).
    ``hyper_connections`` keeps ``streams`` copies of the residual: a sublayer reads
    u = sum_s in[s] x_s, and x_t <- sum_s mix[s, t] x_s + out[t] f(norm(u)) for all streams at once
    (tensors ``<layer>.<mixer_hyper_name>.{in,out,mix}`` and the same for the feed-forward, which
    may be None)."""
    kind: str = "pre_norm"
    mixer: PartSpec = None
    feed_forward: PartSpec = None
    mixer_norm: PartSpec = None
    ff_norm: PartSpec = None
    mixer_post_norm: PartSpec = None       # (sandwich_norm)
    ff_post_norm: PartSpec = None
    # checkpoint names of the parts under the layer's prefix
    mixer_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn"
    ff_norm_name: str = "post_attention_layernorm"
    feed_forward_name: str = "mlp"
    mixer_post_norm_name: str = "post_mixer_norm"
    ff_post_norm_name: str = "post_ff_norm"
    streams: int = 1                       # (hyper_connections)
    mixer_hyper_name: str = "hc1"
    ff_hyper_name: str = "hc2"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``layer``      index into ``ModelSpec.layers`` (weights and parts).  A layer may
                   be named by several runs; they share its weights, and each run
                   that owns a cache gets one of its own.
    ``cache_of``   index of an EARLIER RUN whose cache this run reads instead of
                   owning one: such a run writes no keys, values or state.  None
                   means the run owns (and fills) its cache.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build a model; no family-specific keys."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[BlockSpec, ...]
    run_order: Tuple[LayerRun, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = ()
    # a position encoding that acts on the embedded tokens (learned or sinusoidal
    # absolute positions); encodings that act inside a mixer belong to its spec
    embedding_position: PartSpec = field(default_factory=NoPositionSpec)
    embedding_position_prefix: str = "model.embed_positions"
    # checkpoint naming: prefix of layer i is layer_prefix.format(i)
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm"
    layer_prefix: str = "model.layers.{}"
    # checkpoint tensors that may be present and are ignored
    ignored_suffixes: Tuple[str, ...] = ("rotary_emb.inv_freq",)
    # arithmetic around the layers that some architectures have; None: not applied
    embedding_scale: Optional[float] = None      # embedded tokens are multiplied by it
    embedding_norm: Optional[PartSpec] = None    # an RMS norm on the embedded tokens
    embedding_norm_prefix: str = "model.embed_norm"
    # a number: the residual is kept as that many streams [tokens, streams, hidden], all equal to the
    # embedding at the start and summed before the final norm (blocks of kind hyper_connections)
    residual_streams: Optional[int] = None
    logit_scale: Optional[float] = None          # logits are multiplied by it ...
    logit_softcap: Optional[float] = None        # ... and then become cap * tanh(logits / cap)
