"""Architecture-neutral description of a decoder: what the engine builds from.

An architecture's typed configuration turns its own config.json keys into a
``ModelPlan``.  The plan names, layer by layer, which mixer, feed-forward, norm
and position encoding a block has and with which sizes and constants; the
engine looks each ``kind`` up in the part registries and never asks which
architecture it is running.  The order in which layers run is data as well
(``schedule``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class NormSpec:
    kind: str            # registry key, e.g. "rmsnorm"; "rmsnorm_offset": the tensor holds the scale minus one
    width: int
    eps: float
    weight: str          # tensor name of the scale vector


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # e.g. "rope_split_half"
    rotary_dim: int
    theta: float
    max_positions: int


@dataclass(frozen=True)
class AttentionNames:
    """Tensor names of an attention layer, after the spec's prefix.  An architecture whose checkpoint
    names them otherwise passes its own table; the part knows no name by itself."""
    q: str = "q_proj"
    k: str = "k_proj"
    v: str = "v_proj"
    o: str = "o_proj"
    weight: str = ".weight"
    bias: str = ".bias"


@dataclass(frozen=True)
class SwiGluNames:
    """Tensor names of a SwiGLU MLP, after its prefix."""
    gate: str = "gate_proj.weight"
    up: str = "up_proj.weight"
    down: str = "down_proj.weight"


@dataclass(frozen=True)
class MoeNames:
    """Tensor names of a sparse block, after the spec's prefix; ``expert`` is a template over the expert's index."""
    router: str = "gate.weight"
    shared_gate: str = "shared_expert_gate.weight"
    shared: str = "shared_expert."
    expert: str = "experts.{e}."
    mlp: SwiGluNames = SwiGluNames()


@dataclass(frozen=True)
class AttentionSpec:
    """Softmax attention over cached keys and values with grouped query heads."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qkv_bias: bool
    out_bias: bool
    window: Optional[int]            # None: every earlier key; W: the query and W-1 predecessors
    position: Optional[PositionSpec]
    prefix: str                      # tensor-name prefix, e.g. "model.layers.3.self_attn."
    kind: str = "attention"
    names: AttentionNames = AttentionNames()


@dataclass(frozen=True)
class DenseFfnSpec:
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "swiglu"
    names: SwiGluNames = SwiGluNames()


@dataclass(frozen=True)
class Relu2FfnSpec:
    """down(relu(up h)^2), no biases."""
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "relu2"
    up: str = "up"
    down: str = "down"


@dataclass(frozen=True)
class MoeFfnSpec:
    """Softmax router, top-k routed SwiGLU experts, one shared SwiGLU expert
    scaled by a sigmoid gate (``shared_intermediate`` None: no shared expert).

    ``identity_experts``: the router has that many outputs more than there are experts with weights; an expert
    chosen among them returns its input (times its routing weight).  ``correction``: the name of a tensor with one
    number per router output that is added to the score for the choice only; the weights stay the scores.
    ``groups`` / ``keep_groups``: the router's outputs form that many equal groups of neighbours, a group's score is
    its largest corrected score, and only experts of the best ``keep_groups`` groups can be chosen."""
    hidden: int
    num_experts: int
    top_k: int
    norm_topk: bool
    expert_intermediate: int
    shared_intermediate: Optional[int]
    prefix: str
    kind: str = "moe_swiglu_shared"
    names: MoeNames = MoeNames()
    identity_experts: int = 0
    correction: Optional[str] = None
    groups: int = 0
    keep_groups: int = 0


@dataclass(frozen=True)
class ScaledRopeSpec:
    """Split-half rotary encoding whose slow frequencies are interpolated (YaRN): with ``factor`` None the plain
    frequencies theta^(-2i/d).  Else pair i keeps its frequency while i lies below the pair that makes ``fast``
    turns within ``original`` positions, is divided by ``factor`` beyond the pair that makes ``slow`` turns, with
    a linear ramp between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    rotary_dim: int
    theta: float
    factor: Optional[float] = None
    original: Optional[float] = None
    fast: Optional[float] = None
    slow: Optional[float] = None
    kind: str = "rope_split_half_scaled"


@dataclass(frozen=True)
class LatentAttentionNames:
    """Tensor names of an attention layer with low-rank queries and a cached latent, after the spec's prefix."""
    q_down: str = "dq"
    q_norm: str = "dq.norm"
    q_up: str = "uq"
    kv_down: str = "dkv"
    kv_norm: str = "dkv.norm"
    k_up: str = "uk"
    v_up: str = "uv"
    o: str = "o"
    q: str = "q"                     # full-rank queries (q_rank None)
    head_gate: str = "g"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are up-projections of one cached latent per position; the keys have,
    besides, one rotated part that is the same for every head.  Per head: ``nope_dim`` unrotated and ``rot_dim`` rotated query/key
    channels, ``value_dim`` value channels.  ``q_rank`` None: the queries are one full-rank projection of the layer's
    input.  ``rot_dim`` 0 with ``position`` None: no rotated part and no positions at all.  ``head_gate``: every head's
    output is multiplied by the sigmoid of one number per token and head, a projection of the layer's input."""
    hidden: int
    num_heads: int
    nope_dim: int
    rot_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float                     # multiplies the scores as given
    window: Optional[int]            # None: every earlier key; W: the query and W-1 predecessors
    keep_window: Optional[int]       # how far back the cache has to reach for every layer that reads it
    eps: float                       # of the two latent norms
    position: Optional[ScaledRopeSpec]
    own_kv: bool                     # False: the layer has no down-projection and reads another layer's cache
    prefix: str
    kind: str = "latent_attention"
    names: LatentAttentionNames = LatentAttentionNames()
    head_gate: bool = False


@dataclass(frozen=True)
class GatedRecurrenceNames:
    """Tensor names of the two gated linear recurrences, after the spec's prefix."""
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    norm: str = "norm"
    gate: str = "g"                  # output gate (decay form)
    forget: str = "f"                # forget gate's projection (lower-bound form); its bias is forget + ".b"
    lower: str = "lower"
    receptance: str = "r"
    decay_in: str = "w1"
    decay_out: str = "w2"
    decay_bias: str = "w0"
    bonus: str = "u"
    shift: str = "mu."               # + one of r, k, v, g, w


@dataclass(frozen=True)
class LowerBoundRecurrenceSpec:
    """Gated linear recurrence with one gate for forgetting and writing: what a state row keeps, f_t, and what it
    takes of the new value, 1 - f_t, add up to one, and f_t has a floor per channel:
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T silu(q_t); RMS norm per head, one weight vector for all heads."""
    hidden: int
    num_heads: int
    key_dim: int
    value_dim: int
    eps: float
    prefix: str
    kind: str = "hgrn2"
    names: GatedRecurrenceNames = GatedRecurrenceNames()


@dataclass(frozen=True)
class DecayBonusRecurrenceSpec:
    """Time mixing with token shift, a data-dependent decay per key channel from a low-rank projection, and an
    extra weight u on the token being read: o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_(t-1) + k_t v_t^T;
    per-head unit RMS, a weight per channel and a SiLU gate."""
    hidden: int
    num_heads: int
    head_dim: int
    decay_rank: int
    eps: float
    prefix: str
    kind: str = "wkv"
    names: GatedRecurrenceNames = GatedRecurrenceNames()


@dataclass(frozen=True)
class XieluFfnSpec:
    """down(xIELU(up h)) with the activation's two learned numbers in one tensor."""
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "xielu"
    up: str = "up"
    down: str = "down"
    act: str = "act"


@dataclass(frozen=True)
class DepthMixBlockSpec:
    """Pre-norm layer whose two results are scaled channel by channel (times ``residual_mult``) before they
    join the residual stream, and whose successor gets a weighted sum of the embedding output and every
    layer's result so far (``index`` counts the layers from 0; the weights tensor has index + 2 entries)."""
    mixer: Any
    ffn: Any                         # None: no feed-forward (and no second norm or scale)
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    residual_mult: float
    mixer_scale: str                 # tensor names
    ffn_scale: Optional[str]
    depth_weights: str
    index: int
    depth: int                       # layers of the model
    hidden: int
    kind: str = "prenorm_scaled_depthmix"


@dataclass(frozen=True)
class HashedBigramSpec:
    """A second table whose row is a hash of the token and the token before it:
    row = (previous * mul_prev + token * mul_cur) mod buckets; a sequence's first token reads row ``buckets``
    (the table has buckets + 1 rows)."""
    buckets: int
    mul_prev: int
    mul_cur: int
    weight: str


@dataclass(frozen=True)
class SummedEmbeddingSpec:
    """What enters the residual stream: the token's row, plus (optionally) a hashed bigram row and a sinusoidal
    position vector (entry 2i sin(p b^(-2i/width)), entry 2i + 1 its cosine)."""
    width: int
    bigram: Optional[HashedBigramSpec] = None
    sinusoid_base: Optional[float] = None
    kind: str = "summed"


@dataclass(frozen=True)
class QueryTemperature:
    """Queries at position p are multiplied by 1 + coef ln(floor((p + 1) / every) + 1)."""
    coef: float
    every: int


@dataclass(frozen=True)
class NormedAttentionNames:
    """Tensor names of an attention layer with query/key norms, after the spec's prefix; a bias is the
    projection's name + ``bias``."""
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    bias: str = ".b"
    q_norm: str = "q.norm"
    k_norm: str = "k.norm"


@dataclass(frozen=True)
class NormedAttentionSpec:
    """Causal softmax attention without rotation: queries and keys get an RMS norm per head (one weight vector for
    all heads), keys and values may have different sizes, the scores are multiplied by ``scale`` as given, and
    with ``sink`` the softmax's denominator holds one more term exp(0) that carries no value."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    eps: float
    qkv_bias: bool
    sink: bool
    q_temp: Optional[QueryTemperature]
    window: Optional[int]
    prefix: str
    kind: str = "attention_qknorm"
    names: NormedAttentionNames = NormedAttentionNames()


@dataclass(frozen=True)
class MatrixMemoryNames:
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    gate: str = "g"
    norm: str = "norm"
    input_gate: str = "i"            # its bias is the name + ".b"
    forget_gate: str = "f"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """Matrix memory with an exponential input gate and a sigmoid forget gate, both soft-capped, kept in range by
    a running maximum m (m_0 = 0):  m_t = max(f_t + m_(t-1), i_t);  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) +
    e^(i_t - m_t) k_t v_t^T, n_t likewise with k_t alone;  o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6);
    each head's o is scaled to unit root mean square, then a weight per channel and a sigmoid gate."""
    hidden: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    prefix: str
    kind: str = "mlstm"
    names: MatrixMemoryNames = MatrixMemoryNames()


@dataclass(frozen=True)
class GatedDiagonalNames:
    gate_branch: str = "y"           # biases: the name + ".b"
    in_branch: str = "x"
    conv: str = "conv"
    recurrence_gate: str = "ra"
    input_gate: str = "ri"
    decay: str = "lam"
    o: str = "o"


@dataclass(frozen=True)
class GatedDiagonalSpec:
    """Two branches of ``channels``: a GELU gate, and a causal convolution of ``taps`` per channel followed by a
    diagonal recurrence whose decay a_t = exp(-c r_t softplus(lam)) and input gate come from block-diagonal
    projections of the convolution's output:  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t."""
    hidden: int
    channels: int
    blocks: int
    taps: int
    decay_scale: float               # c above
    prefix: str
    kind: str = "rglru"
    names: GatedDiagonalNames = GatedDiagonalNames()


@dataclass(frozen=True)
class ScaledInputMoeSpec:
    """Sigmoid router; the ``top_k`` experts with the largest scores; a chosen expert's score multiplies its
    input; experts are down(act(up x)) with ``activation`` ("relu2": the square of relu); an optional shared
    expert of the same form takes every token."""
    hidden: int
    num_experts: int
    top_k: int
    expert_intermediate: int
    shared_intermediate: Optional[int]
    prefix: str
    activation: str = "relu2"
    kind: str = "moe_sigmoid_scaled_input"
    router: str = "router"
    expert: str = "e{e}."
    shared: str = "shared."
    up: str = "up"
    down: str = "down"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x += norm_after(mixer(norm_before(x))); x += norm_after(ffn(norm_before(x))): every sublayer's result is
    normalised before it joins the residual stream.  ``ffn`` None: the layer has a mixer only."""
    mixer: Any
    ffn: Any
    mixer_norm: NormSpec
    mixer_post_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    ffn_post_norm: Optional[NormSpec]
    kind: str = "sandwich_residual"


@dataclass(frozen=True)
class WideNormAttentionNames:
    """Tensor names of an attention layer whose query and key norms span the whole projection, after the spec's prefix."""
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    q_norm: str = "q.norm"
    k_norm: str = "k.norm"
    sink: str = "sink"


@dataclass(frozen=True)
class WideNormAttentionSpec:
    """Causal softmax attention over cached keys and values with grouped query heads, where the RMS norm of the
    queries (and of the keys) runs over the whole projection, all heads at once, with a weight per channel, before the
    rotation; the rotation (``position``, split-half pairs) covers the first channels of every head; scores are
    multiplied by ``scale`` as given; keys and values may have different sizes.  Which keys a query sees: every
    earlier one, the last ``window``, or (``chunk``) those of its own block of ``chunk`` positions counted from the
    sequence's start.  ``learned_sink``: the softmax's denominator holds one more term exp(sink_h), a learned number
    per head that is not scaled and carries no value."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    eps: float
    learned_sink: bool
    window: Optional[int]
    chunk: Optional[int]
    position: Optional[ScaledRopeSpec]
    prefix: str
    kind: str = "attention_widenorm"
    names: WideNormAttentionNames = WideNormAttentionNames()


@dataclass(frozen=True)
class GatedDeltaNames:
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    conv: str = ".conv"              # after q, k or v
    beta: str = "b"
    decay_log: str = "A_log"
    decay_in: str = "a1"
    decay_out: str = "a2"
    decay_bias: str = "dt_bias"
    gate_in: str = "g1"
    gate_out: str = "g2"
    norm: str = "norm"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Delta rule with a decay per head and key channel.  q, k (``num_kv_heads`` heads of ``key_dim``) and v
    (``num_heads`` heads of ``value_dim``) pass a causal convolution of ``taps`` per channel and SiLU; q and k become unit
    vectors per head (x / sqrt(sum x^2 + unit_eps)), q times key_dim^(-1/2);  beta = sigmoid(W_b h) per head;
    d = exp(-exp(A_h) softplus(W_a2 W_a1 h + bias)) per head and key channel.  Per head, in this order:
    S <- diag(d) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Each head's o is scaled to unit root mean
    square (``eps``), times a weight per value channel shared by the heads, times sigmoid(W_g2 W_g1 h); then W_o.
    Value head h reads query/key head h // (num_heads / num_kv_heads).  The two inner widths come from the tensors."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    taps: int
    decay_rank: int
    gate_rank: int
    eps: float
    prefix: str
    unit_eps: float = 1e-6
    kind: str = "gated_delta"
    names: GatedDeltaNames = GatedDeltaNames()


@dataclass(frozen=True)
class ChannelDecayAttentionNames:
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    gate: str = "g"
    norm: str = "norm"
    decay_in: str = "a1"
    decay_out: str = "a2"
    decay_bias: str = "a2.b"


@dataclass(frozen=True)
class ChannelDecayAttentionSpec:
    """Gated linear attention: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head with q = W_q h
    key_dim^(-1/2) and a_t = sigmoid(W_a2 W_a1 h + bias)^(1/tau) per head and key channel; every head's o is RMS-normed
    with a weight per value channel shared by the heads, the heads' concatenation is multiplied by silu(W_g h),
    then W_o.  The decay's inner width comes from the tensors."""
    hidden: int
    num_heads: int
    key_dim: int
    value_dim: int
    tau: float
    decay_rank: int
    eps: float
    prefix: str
    kind: str = "gla"
    names: ChannelDecayAttentionNames = ChannelDecayAttentionNames()


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input; the result is sum_i scales[i] * branches[i](h)."""
    hidden: int
    branches: tuple                  # mixer specs
    scales: tuple                    # one number per branch
    kind: str = "parallel_sum"


@dataclass(frozen=True)
class ClampedGluFfnSpec:
    """down(g sigmoid(alpha g) (u + up_shift)) with g = min(gate h, limit) and u = clamp(up h, -limit, limit)."""
    hidden: int
    intermediate: int
    limit: float
    prefix: str
    alpha: float = 1.702
    up_shift: float = 1.0
    kind: str = "glu_clamped"
    names: SwiGluNames = SwiGluNames("gate", "up", "down")


@dataclass(frozen=True)
class HyperConnectionNames:
    """Tensor names of one sublayer's connection weights, after its prefix."""
    read: str = "in"
    write: str = "out"
    mix: str = "mix"


@dataclass(frozen=True)
class HyperConnectionBlockSpec:
    """A pre-norm layer over ``streams`` copies of the residual stream x_1 .. x_s (all equal to what enters the
    stack).  A sublayer reads u = sum_s in[s] x_s, computes y = sublayer(norm(u)), and writes, all streams at once
    from the old ones, x_t <- sum_s mix[s, t] x_s + out[t] y.  Behind the stack's last layer the streams are summed.
    ``index`` counts the layers of the stack from 0, ``depth`` is their number."""
    mixer: Any
    ffn: Any                         # None: the layer has a mixer only
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    streams: int
    mixer_prefix: str                # e.g. "l3.hc1."
    ffn_prefix: Optional[str]
    index: int
    depth: int
    hidden: int
    kind: str = "hyper_connections"
    names: HyperConnectionNames = HyperConnectionNames()


@dataclass(frozen=True)
class NeighbourRopeSpec:
    """Rotary encoding over neighbouring channels: of the first ``rotary_dim`` channels of a head, channel 2i is
    rotated with channel 2i + 1 by the angle position * theta^(-2i / rotary_dim)."""
    rotary_dim: int
    theta: float
    factor: Optional[float] = None   # no interpolation in this form
    kind: str = "rope_neighbour_pairs"


@dataclass(frozen=True)
class UnitNormAttentionNames:
    q: str = "q"
    k: str = "k"
    v: str = "v"
    o: str = "o"
    bias: str = ".b"
    sink: str = "sink"
    value_blend: str = "vmix"


@dataclass(frozen=True)
class UnitNormAttentionSpec:
    """Causal softmax attention over cached keys and values with grouped query heads: projections with optional
    biases; rotation of neighbouring channel pairs of the first channels of every head (``position``); then, with
    ``unit_heads``, queries and keys divided by their root mean square per head (no weight); scores times ``scale``
    as given; a window; ``learned_sink``: one more term exp(sink_h) per head in the softmax's denominator, unscaled,
    without a value.  ``value_blend``: "first" marks the layer whose values (of the step's tokens) later layers
    blend with; "blend": v <- (1 - lambda) v + lambda v_first with lambda a learned number, and the blended values
    are what the cache holds; None: neither.  A "first" layer still names lambda's tensor (a checkpoint holds it)."""
    hidden: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    eps: float
    qkv_bias: bool
    unit_heads: bool
    learned_sink: bool
    window: Optional[int]
    position: Optional[NeighbourRopeSpec]
    value_blend: Optional[str]
    prefix: str
    kind: str = "attention_unitnorm"
    names: UnitNormAttentionNames = UnitNormAttentionNames()


@dataclass(frozen=True)
class SelectiveScanNames:
    in_proj: str = "in"
    conv: str = "conv"
    conv_bias: str = "conv.b"
    x_proj: str = "x"
    dt_proj: str = "dt"
    dt_bias: str = "dt.b"
    a_log: str = "A_log"
    skip: str = "D"
    o: str = "o"


@dataclass(frozen=True)
class SelectiveScanSpec:
    """W_in h = [x | z] of ``inner`` channels each; x passes a causal convolution of ``taps`` per channel with a bias,
    then SiLU; W_x x = [dt_low (dt_rank) | B (state) | C (state)]; dt = softplus(W_dt dt_low + bias) per channel;
    per channel c and state entry n: S <- exp(-dt exp(a_log[c, n])) S + dt x_c B_n; y_c = S[c] . C + skip_c x_c; the
    result times silu(z), then W_o."""
    hidden: int
    inner: int
    state: int
    dt_rank: int
    taps: int
    prefix: str
    kind: str = "selective_scan"
    names: SelectiveScanNames = SelectiveScanNames()


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts it has and how they are arranged.  ``ffn`` (and ``ffn_norm``) None: a mixer only."""
    mixer: Any                       # any spec object with a ``kind``
    ffn: Any
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    kind: str = "prenorm_residual"   # x += mixer(norm(x)); x += ffn(norm(x))


@dataclass(frozen=True)
class ScheduleEntry:
    """One call of a layer.  ``cache_of`` names an earlier schedule index whose
    cache this call reads instead of holding one of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelPlan:
    architecture: str
    hidden: int
    vocab: int
    max_positions: int
    blocks: list
    schedule: list
    final_norm: NormSpec
    embed_weight: str
    head_weight: Optional[str]       # None: the head is the embedding table
    stop_token_ids: tuple = ()
    # tensor names that a checkpoint may hold although nothing reads them
    tolerated_suffixes: tuple = ()
    extra: dict = field(default_factory=dict)
    # the two ends of the model, as far as they are more than a lookup and a product:
    embed_scale: float = 1.0                 # the table's rows are multiplied by this as they enter the residual stream
    logit_softcap: Optional[float] = None    # logits = cap * tanh(logits / cap)
    tied_head_name: Optional[str] = None     # with head_weight None: a checkpoint may still carry the head under this name
    embedding: Any = None                    # None: the token's row alone; else a spec of the ``embedding`` family
