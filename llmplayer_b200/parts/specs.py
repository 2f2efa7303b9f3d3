"""Descriptions of the parts a decoder is put together from.

A specification is plain data: it carries every size, constant and tensor name
its part needs, and a ``kind`` that the part registries resolve to a class.
An architecture turns its configuration into a :class:`ModelLayout`; nothing
below that layout knows which architecture it came from.

The reference describes the same pieces by fields of one configuration object
(model/ModelConfig.java:100-156) and wires them in code
(inference/InferenceEngine.java:53-101, inference/TransformerBlock.java:64-159).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

# Kinds of tensors: they decide how random weights are drawn and how a tensor
# is held on the device.
MATRIX = "matrix"   # [out, in] weight of a linear map, or an embedding table
GAIN = "gain"       # per-feature multiplier of a norm, drawn around one
INTEGER = "integer"  # integer table, held as int32
BIAS = "bias"       # additive vector or a handful of learned numbers, drawn around zero, used in float32


ANY = -1            # a size that the model file decides: the loader accepts whatever it finds there


@dataclass(frozen=True)
class TensorSpec:
    """Shape and kind of one named tensor of a model folder. A size of ``ANY`` is read off the file
    (``fill`` is what a writer of random weights puts there)."""
    shape: Tuple[int, ...]
    kind: str = MATRIX
    fill: int = 16

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(w == ANY or w == g for w, g in zip(self.shape, shape))

    def concrete(self) -> Tuple[int, ...]:
        return tuple(self.fill if w == ANY else w for w in self.shape)


@dataclass(frozen=True)
class NormSpec:
    """``kind="rmsnorm"``: x / sqrt(mean(x^2) + eps) * weight. ``kind="layernorm"``: (x - mean) /
    sqrt(variance + eps) * weight, the variance being the mean squared deviation; no bias."""
    size: int
    eps: float
    weight: str
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency-dependent stretching of rotary wavelengths ("llama3" rope_scaling)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position: int


@dataclass(frozen=True)
class YarnScaling:
    """Stretching of rotary frequencies by how many turns a pair makes over the ``original`` context ("YaRN"). With
    turn(t) = dims * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turn(fast)), 0), hi = min(ceil(turn(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i rotates by f_i / factor * ramp_i +
    f_i * (1 - ramp_i), and cosine and sine are both multiplied by 0.1 * ln(factor) + 1."""
    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    ``kind="rope"`` rotates the first ``rotary_dim`` features of each head;
    ``pairing`` is ``"split_half"`` (feature i with i + rotary_dim/2) or
    ``"interleaved"`` (2i with 2i+1). ``kind="none"`` leaves them as they are.
    ``scaling``: a :class:`Llama3Scaling` or a :class:`YarnScaling`.
    """
    kind: str = "rope"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 0.0
    scaling: Optional[object] = None
    pairing: str = "split_half"


@dataclass(frozen=True)
class AttentionSpec:
    """Softmax attention over the cached keys of a sequence, with grouped query heads.

    ``window`` limits a query at position p to keys at positions > p - window
    (None: all keys). ``shares_kv`` marks a layer that projects no keys or
    values and attends over the cache of the schedule entry it is pointed at.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    q: str
    o: str
    k: Optional[str] = None
    v: Optional[str] = None
    window: Optional[int] = None
    shares_kv: bool = False
    kind: str = "attention"
    # What a layer may have beyond that (a layer with any of these takes the general path of the mixer):
    value_dim: Optional[int] = None      # size of a value head when it differs from head_dim (``o`` is [hidden, heads * value_dim])
    q_bias: Optional[str] = None         # additive vectors of the three projections
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    unit_norm_eps: Optional[float] = None    # after the rotation, queries and keys are divided by their root mean square per head
    softcap: Optional[float] = None      # score <- softcap * tanh(score / softcap), after the scale
    sink: Optional[str] = None           # tensor [heads]: a learned logit per head in the softmax's denominator, without key or value
    exact_weights: bool = False          # softmax weights meet the values at float32 precision also on the tensor cores
    q_norm: Optional[str] = None         # gains [head_dim], shared by the heads: BEFORE the rotation every query / key head is
    k_norm: Optional[str] = None         # RMS-normed over head_dim with that gain and ``qk_norm_eps`` inside the root
    qk_norm_eps: float = 0.0
    o_bias: Optional[str] = None         # additive vector [hidden] of the output projection
    sink_value: Optional[float] = None   # a constant logit (the same for every head) in the softmax's denominator: 0.0 adds one to it
    # The window that the layer's cache must keep (None: everything) when layers that attend over this layer's keys look
    # further back than the layer itself; "own": the layer's own ``window``.
    cache_window: object = "own"
    keep_first: Optional[int] = None     # with ``window``: a sequence's first so many tokens stay visible to every later query, at their true positions

    @property
    def general(self) -> bool:
        return (bool(self.keep_first) or self.value_dim not in (None, self.head_dim) or any(b is not None for b in (self.q_bias, self.k_bias, self.v_bias))
                or self.unit_norm_eps is not None or self.softcap is not None or self.sink is not None or self.exact_weights
                or self.q_norm is not None or self.k_norm is not None or self.o_bias is not None or self.sink_value is not None)


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate x) * (up x))."""
    hidden_size: int
    intermediate_size: int
    gate: str
    up: str
    down: str
    kind: str = "swiglu"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are linear maps of one cached low-rank latent per position.

    The down projection ``kv_down`` yields ``kv_rank + rope_dim`` values: the first ``kv_rank``, RMS-normed
    with ``latent_norm``, are the latent; the rest are one rotated key part shared by all heads. Head h's
    unrotated key is ``k_up`` [h] times the latent, its value ``v_up`` [h] times the latent; a query head is
    laid out [``nope_dim`` unrotated | ``rope_dim`` rotated]. ``position`` rotates the ``rope_dim`` part.
    ``out_gate`` (optional): a matrix [heads, hidden] whose sigmoid scales each head's output.
    ``q_down`` / ``q_norm`` (optional, together): queries go through a latent of their own, q = ``q`` rms_norm(``q_down`` x)
    with the gain ``q_norm``; ``q`` is then [heads * (nope + rope), q_rank], the rank read off ``q_down``'s config size
    ``q_rank``. ``window``: a query at position p sees keys p - window + 1 .. p (None: all earlier keys).
    """
    hidden_size: int
    num_heads: int
    nope_dim: int
    rope_dim: int
    value_dim: int
    kv_rank: int
    scale: float
    norm_eps: float
    position: PositionSpec
    q: str
    kv_down: str
    latent_norm: str
    k_up: str
    v_up: str
    o: str
    out_gate: Optional[str] = None
    kind: str = "latent_attention"
    q_down: Optional[str] = None
    q_norm: Optional[str] = None
    q_rank: int = 0
    window: Optional[int] = None
    exact_weights: bool = False          # prompts run as ordinary heads: softmax weights meet the values at float32 precision


@dataclass(frozen=True)
class LowRankDecaySpec:
    """A decay per key channel from the layer's input: sigmoid(up(down(x)) + bias)^(1 / temperature).
    The width of the factor is read off ``down``'s shape."""
    temperature: float
    down: str
    up: str
    bias: str


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a matrix state per head, S <- diag(decay) S + k v^T, o = S^T q, queries
    scaled by ``key_dim`` ** -0.5; each head's output is RMS-normed over ``value_dim`` with the shared gain
    ``out_norm``, multiplied by silu(``gate`` x) and projected by ``o``."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    norm_eps: float
    decay: LowRankDecaySpec
    q: str
    k: str
    v: str
    gate: str
    out_norm: str
    o: str
    kind: str = "gated_linear_attention"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """A matrix memory per head with exponential gates and a running maximum (the mLSTM of the xLSTM family):
    with i = cap * tanh((W_i x + b_i) / cap), f = logsigmoid(cap * tanh((W_f x + b_f) / cap)) per head,
    m_t = max(f + m_(t-1), i) (m starts at ``0``), S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t the same
    with k alone, and o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6) with q scaled by ``key_dim`` ** -0.5. Each head's o
    is divided by its root mean square, the heads are multiplied by the gain ``out_norm`` [heads * value_dim] and by
    sigmoid(``gate`` x), and projected by ``o``. ``gate_cap`` None: the gates' pre-activations are not capped."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    norm_eps: float
    gate_cap: Optional[float]
    q: str
    k: str
    v: str
    gate: str
    input_gate: str
    input_gate_bias: str
    forget_gate: str
    forget_gate_bias: str
    out_norm: str
    o: str
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class StateSpaceSpec:
    """A selective state space per head behind a short convolution (the state-space-duality form, "Mamba-2"). With
    inner = heads * head_dim, N = state_dim, G = groups, ``in_proj`` x is laid out [z: inner | x: inner | B: G N | C: G N |
    dt: heads]. x, B and C together pass a causal convolution per channel (``conv`` [inner + 2 G N, taps], bias
    ``conv_bias``, the last tap on the token itself) and silu. dt = softplus(dt + ``dt_bias``) without a clamp; per head
    (head h reads group h // (heads // groups)), S_t = exp(-exp(``a_log``[h]) dt) S_(t-1) + dt B_t x_t^T (S: [N, head_dim]),
    y_t = S_t^T C_t + ``skip``[h] x_t. y (heads side by side) is multiplied by silu(z), then divided in ``norm_groups``
    equal parts by each part's root mean square (``norm_eps`` inside the root), times ``out_norm`` [inner], then ``o``.
    The state and the convolution's last taps - 1 inputs are float32 and start at zero."""
    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    in_proj: str
    conv: str
    conv_bias: str
    dt_bias: str
    a_log: str
    skip: str
    out_norm: str
    o: str
    kind: str = "state_space"


@dataclass(frozen=True)
class GatedDeltaRuleSpec:
    """A matrix state per head updated by the gated delta rule. q = ``q`` x and k = ``k`` x have ``num_qk_heads`` heads of
    ``key_dim``, v = ``v`` x has ``num_heads`` heads of ``value_dim`` (head h reads query / key head h // (num_heads //
    num_qk_heads)); each passes a short causal convolution per channel (``q_conv`` / ``k_conv`` / ``v_conv`` [channels,
    taps], no bias) and silu. q and k become unit vectors per head, x / sqrt(sum(x^2) + 1e-6), q also times key_dim^-1/2.
    Per head: strength = sigmoid(``strength`` x), decay = exp(-exp(``a_log``) softplus(``decay`` x + ``dt_bias``));
    S <- decay S; u = strength (v - S^T k); S <- S + k u^T; o = S^T q. Each head's o is divided by its root mean square
    over value_dim (``norm_eps``), times ``out_norm`` [value_dim] (shared by the heads), times silu(``gate`` x); then ``o``.
    The state and the convolutions' last inputs are float32 and start at zero."""
    hidden_size: int
    num_heads: int
    num_qk_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    q: str
    k: str
    v: str
    q_conv: str
    k_conv: str
    v_conv: str
    strength: str
    decay: str
    a_log: str
    dt_bias: str
    gate: str
    out_norm: str
    o: str
    kind: str = "gated_delta_rule"


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers side by side that read the same input: ``left_scale`` * left(x) + ``right_scale`` * right(x). Each
    keeps its own cache or state."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "mixer_pair"


@dataclass(frozen=True)
class TimeMixSpec:
    """Time mixing with a matrix state per head and a decay per key channel that depends on the token (the WKV
    recurrence of the RWKV family, version 6). With x' the previous token's input (zeros before a sequence's first
    token), each of r, k, v, g, w reads its own blend x + (x' - x) * mu_s (``mu`` + "r", "k", "v", "g", "w"; [hidden]
    each). r, k, v = ``r`` / ``k`` / ``v`` of their blends ([heads * head_dim, hidden]); the output gate is
    silu(``gate`` blend_g); the decay is exp(-exp(``decay_up`` tanh(``decay_down`` blend_w) + ``decay_bias``)) per head
    and key channel (the width of the factor is read off ``decay_down``). Per head, with the bonus ``bonus``
    [heads, head_dim]:

        o_t = (S_(t-1) + diag(bonus) k_t v_t^T)^T r_t;    S_t = diag(decay_t) S_(t-1) + k_t v_t^T

    Each head's o_t is divided by its root mean square (``norm_eps`` inside the root), the heads are multiplied by the
    gain ``out_norm`` [heads * head_dim] and by the gate, and projected by ``o``. The state (S and the previous token's
    input) is float32 and starts at zero."""
    hidden_size: int
    num_heads: int
    head_dim: int
    norm_eps: float
    mu: str
    r: str
    k: str
    v: str
    gate: str
    decay_down: str
    decay_up: str
    decay_bias: str
    bonus: str
    out_norm: str
    o: str
    kind: str = "time_mix"


@dataclass(frozen=True)
class GatedDenseSpec:
    """Dense gated feed-forward down(act(gate x + b_g) * (up x + b_u)) + b_d with ``activation`` "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) or "silu"; the additive vectors are optional."""
    hidden_size: int
    intermediate_size: int
    gate: str
    up: str
    down: str
    gate_bias: Optional[str] = None
    up_bias: Optional[str] = None
    down_bias: Optional[str] = None
    activation: str = "gelu_tanh"
    kind: str = "gated_dense"


@dataclass(frozen=True)
class SquaredReLUSpec:
    """Dense feed-forward down(relu(up x)^2)."""
    hidden_size: int
    intermediate_size: int
    up: str
    down: str
    kind: str = "squared_relu"


@dataclass(frozen=True)
class ExpertRoutingSpec:
    """How a token chooses its experts: scores sigmoid(router x); the experts form ``groups`` equal groups of
    neighbours whose score is the sum of their two largest scores; only experts of the ``keep_groups`` best groups
    may be chosen; the ``top`` largest scores among those win, and their weights are the scores divided by their sum.

    ``scoring="softmax_top"``: the ``top`` experts with the largest logits router x + ``router_bias`` are chosen, and
    their weights are the softmax over the chosen logits alone (``groups`` and ``keep_groups`` stay 1).

    ``scoring="softmax_groups"``: scores softmax(router x) over all router outputs: the ``num_experts`` experts and
    ``identity_experts`` further ones without tensors whose output is their input. The choice is made on score +
    ``correction`` [all outputs]; a group's score is its largest choice score, the ``top`` largest choice scores inside
    the ``keep_groups`` best groups win; the weights are the chosen scores (without the correction) times
    ``weight_scale``, not renormalised."""
    num_experts: int
    top: int
    groups: int
    keep_groups: int
    router: str
    scoring: str = "sigmoid_groups"
    router_bias: Optional[str] = None
    correction: Optional[str] = None
    weight_scale: float = 1.0
    identity_experts: int = 0


@dataclass(frozen=True)
class MixtureSpec:
    """Mixture of gated experts down(silu(gate x) * (up x)) without biases. Expert e's tensors are
    ``expert_prefix`` + ``e<e>.`` + gate / up / down. ``shared_size`` > 0: one more expert of that size
    (``shared_prefix`` + gate / up / down) runs for every token with weight one.

    ``activation="clamped"``: an expert is down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate x, limit) and
    u = clamp(up x, -limit, limit); ``limit`` belongs to the routed experts, ``shared_limit`` to the shared one.
    ``shared_gate``: a matrix [1, hidden]; the shared expert's output is multiplied by sigmoid(shared_gate x), one
    number per token."""
    hidden_size: int
    expert_size: int
    routing: ExpertRoutingSpec
    expert_prefix: str
    shared_size: int = 0
    shared_prefix: Optional[str] = None
    kind: str = "mixture"
    activation: str = "silu"
    limit: float = 0.0
    shared_limit: float = 0.0
    shared_gate: Optional[str] = None


@dataclass(frozen=True)
class XIELUSpec:
    """Dense feed-forward down(act(up x)) with the xIELU activation, whose two learned numbers are the
    tensor ``act`` [2]."""
    hidden_size: int
    intermediate_size: int
    up: str
    down: str
    act: str
    kind: str = "xielu"


@dataclass(frozen=True)
class ResidualGateSpec:
    """sigmoid(weight x + bias), one value per feature, multiplying a sublayer's result."""
    weight: str
    bias: str


@dataclass(frozen=True)
class DepthMixSpec:
    """After a layer, the stream becomes a weighted sum of the embedding's output and of every layer's result
    so far: ``weights`` [count] with count = 2 + the number of layers before this one."""
    weights: str
    count: int
    total: int          # streams of the whole model (layers + 1): the size of the buffer all layers share


@dataclass(frozen=True)
class ParallelBlockSpec:
    """One layer with one norm whose output both sublayers read: x + mixer(norm(x)) + ffn(norm(x)).
    ``ffn`` may be None. Each sublayer's result may be gated (:class:`ResidualGateSpec`, from the same
    normed input); ``depth_mix`` replaces the result by a weighted sum over depth."""
    norm: NormSpec
    mixer: object
    ffn: Optional[object] = None
    mixer_gate: Optional[ResidualGateSpec] = None
    ffn_gate: Optional[ResidualGateSpec] = None
    depth_mix: Optional[DepthMixSpec] = None
    kind: str = "parallel"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """One layer with a norm in front of and behind each sublayer:
    x += post_mixer_norm(mixer(mixer_norm(x))); x += post_ffn_norm(ffn(ffn_norm(x))). ``ffn`` may be None (then the
    two norms around it are None as well)."""
    mixer_norm: NormSpec
    mixer: object
    post_mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec] = None
    ffn: Optional[object] = None
    post_ffn_norm: Optional[NormSpec] = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """One layer whose sublayers read the stream itself and whose results are normed before they are added:
    x += mixer_scale * post_mixer_norm(mixer(x)); x += ffn_scale * post_ffn_norm(ffn(x)). The scales (tensors [hidden],
    optional) multiply the normed result element by element (a layer scale). ``ffn`` may be None (then its norm and
    scale are None as well)."""
    mixer: object
    post_mixer_norm: NormSpec
    mixer_scale: Optional[str] = None
    ffn: Optional[object] = None
    post_ffn_norm: Optional[NormSpec] = None
    ffn_scale: Optional[str] = None
    kind: str = "postnorm"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how its norms, mixer and feed-forward are arranged.

    ``kind="prenorm"``: x += mixer(norm(x)); x += feed_forward(norm(x)). ``ffn`` and ``ffn_norm`` may both be None (a
    layer without a feed-forward).
    """
    mixer_norm: NormSpec
    mixer: object
    ffn_norm: Optional[NormSpec]
    ffn: Optional[object]
    kind: str = "prenorm"


@dataclass(frozen=True)
class EmbeddingSpec:
    """The token's row of the table, times ``scale``."""
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "embedding"
    scale: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """Final norm and projection to the vocabulary. ``weight`` may name the
    embedding table (a tied head). ``logit_scale`` multiplies the logits."""
    vocab_size: int
    hidden_size: int
    norm: NormSpec
    weight: str
    kind: str = "linear_head"
    logit_scale: float = 1.0


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``reads_cache_of`` is the index of an earlier entry
    of the schedule whose cache this run attends over instead of keeping its own."""
    layer: int
    reads_cache_of: Optional[int] = None
    # Before the run, added to the stream: the embedding's output (the stream as it entered the first run), and row
    # ``add_row`` of the float32 tensor ``add_vector`` [rows, hidden] (a learned vector per pass of a repeated span)
    add_embedding: bool = False
    add_vector: Optional[str] = None
    add_row: int = 0


@dataclass(frozen=True)
class ModelLayout:
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    head: HeadSpec
    schedule: Tuple[ScheduleEntry, ...] = field(default=())

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        """The schedule, or every layer once in order when none is given."""
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))
