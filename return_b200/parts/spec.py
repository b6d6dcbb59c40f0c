"""Specifications of the parts a decoder is put together from.

A specification is a frozen record of sizes and constants with a ``kind``.  The registries of
``return_b200/parts/registry.py`` map a kind to the class that runs it.  An architecture
(``return_b200/models``) turns its configuration into a ``DecoderSpec``: one ``BlockSpec`` per
layer, chosen layer by layer, and a ``schedule`` that says in which order layers run.  A
specification never names a model; a part built from it does not know which model it is in.

Anything with a ``kind`` attribute can be a specification, so a test or a later architecture
can define its own records for its own parts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (offset + w) over the last ``size`` elements."""
    size: int
    eps: float
    offset: float = 0.0
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split rotary encoding of the first ``rotary_dim`` elements of a head."""
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class ScaledRopeSpec:
    """Half-split rotary encoding of the first ``rotary_dim`` elements of a head whose long wavelengths may be slowed
    down.  ``scaling`` None, or (factor, low, high, original): with wavelength l = 2 pi / f, f is kept where
    l < original / high, divided by factor where l > original / low, and blended linearly in
    s = (original / l - low) / (high - low) between the two.  Tables are worked out in float64."""
    rotary_dim: int
    theta: float
    max_positions: int
    scaling: Optional[Tuple[float, float, float, float]] = None
    kind: str = "rope_scaled"


@dataclass(frozen=True)
class RampedRopeSpec:
    """Half-split rotary encoding of the first ``rotary_dim`` elements whose frequencies are stretched along a ramp over
    the pair index.  With f_i = theta^(-2i / rotary_dim) and index(n) = rotary_dim ln(original / (2 pi n)) / (2 ln theta),
    the ramp runs from lo = max(floor(index(fast)), 0) to hi = min(ceil(index(slow)), rotary_dim - 1):
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), and the frequency is f_i / factor * r_i + f_i * (1 - r_i).  cos and
    sin are multiplied by ``magnitude_slope`` * ln(factor) + 1.  ``factor`` None: plain frequencies, no factor on the
    tables.  Tables are worked out in float64."""
    rotary_dim: int
    theta: float
    max_positions: int
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    magnitude_slope: float = 0.1
    kind: str = "rope_ramped"


@dataclass(frozen=True)
class InterleavedRopeSpec:
    """Rotary encoding of the first ``rotary_dim`` elements of a head in which element 2i is paired with element 2i + 1:
    the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * theta^(-2i / rotary_dim).
    Tables are worked out in float64."""
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_interleaved"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are linear maps of one cached latent a token.  Per head: ``key_dim``
    unrotated query/key elements, ``rot_dim`` rotated ones (the rotated key part is one vector shared by all heads,
    projected beside the latent and not normed), ``value_dim`` value elements; the latent has ``kv_rank`` numbers and is
    RMS-normed (plain weight, ``eps``).  The score is (q . k) * ``scale`` over both parts.  Options: ``q_rank`` (queries
    go through a normed latent of their own), ``window`` (the last n keys, the query's own included), ``sink`` (a learned
    term per head in the softmax's denominator that has no key and no value), ``gate`` (a head's output times the
    logistic of a projection of the mixer's input)."""
    hidden_size: int
    num_heads: int
    key_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    scale: float
    eps: float
    q_rank: Optional[int] = None
    window: Optional[int] = None
    sink: bool = False
    gate: bool = False
    position: Optional[Any] = None        # the encoding of the rotated part (rotary_dim == rot_dim), None if rot_dim == 0
    kind: str = "latent_attention"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    window: Optional[int] = None          # None: every earlier key; n: the last n keys
    qk_norm: Optional[NormSpec] = None    # per-head norm of q and k before the rotation
    position: Optional[Any] = None        # a position-encoding spec, e.g. RopeSpec
    kind: str = "attention"
    # Key and value sizes of the checkpoint's heads where they differ from ``head_dim``: the heads are then padded with
    # zeros to ``head_dim`` when the weights are loaded (zero key elements add nothing to a score, zero value
    # elements meet zero columns of the output projection), so one cache layout and one set of kernels serve them.
    key_dim: Optional[int] = None
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Causal grouped-query attention over a paged cache whose heads are prepared row by row, with an output gate.
    Heads have ``key_dim`` query/key elements and ``value_dim`` value elements (the cache holds both padded to one size).
    Options, each off unless given: ``bias`` (q, k, v projections have biases); ``whole_norm_eps`` (an RMS norm with a
    weight per element over the whole q projection and over the whole k projection, before the rotation);
    ``position`` (an ``InterleavedRopeSpec``: q and k are rotated, values are not); ``values_are_keys`` (there is no value
    projection: a value is the key projection as it comes out of the product, before norm and rotation);
    ``window`` (a query sees the last n keys, its own included) or ``chunk`` (a query sees the earlier keys of its own block
    of n positions, blocks counted from position 0); ``softcap`` (a scaled score s becomes cap tanh(s / cap));
    ``slope_exponent`` e (slope_h (i - j) is taken off the score, slope_h = 2^(-e (h + 1) / heads)); ``sink`` (a learned
    number per head whose exponential joins the softmax's denominator); ``gate`` "head" (a head's output times the
    logistic of one projected number) or "element" (one per value element).  ``own_cache`` False: the layer has no key
    and value projections and reads the cache that another run of the schedule wrote.  ``cache_window``: how many of the
    latest keys the cache must keep for this layer and every layer that reads its cache (None: all)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    bias: bool = False
    whole_norm_eps: Optional[float] = None
    position: Optional[Any] = None
    values_are_keys: bool = False
    window: Optional[int] = None
    chunk: Optional[int] = None
    softcap: Optional[float] = None
    slope_exponent: Optional[float] = None
    sink: bool = False
    gate: Optional[str] = None
    own_cache: bool = True
    cache_window: Optional[int] = None
    kind: str = "gated_attention"


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with one fixed decay a head and no softmax: S <- decay S + k v^T, o = S^T q; q and k are
    rotated (``position``), k is scaled by key_dim^-1/2; each head's o is divided by its root mean square, gated
    by silu of a projection of the input, and projected out."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    eps: float
    position: Optional[Any] = None
    kind: str = "retention"


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """Gated delta rule with a decay per head and key channel.  q, k (``num_kv_heads`` heads) and v pass a causal
    convolution of ``conv_taps`` taps and silu; q and k become unit vectors (``unit_eps`` under the root), q times
    key_dim^-1/2; beta = sigmoid of a projection; the decay is exp(-exp(A_log) softplus(low-rank projection +
    dt_bias)); the read-out is normed per head, weighted, gated by sigmoid of a low-rank projection."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    eps: float
    unit_eps: float = 1e-6
    kind: str = "channel_delta"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule with one decay per head and token.  q, k (``num_kv_heads`` heads of ``key_dim``) and v
    (``num_heads`` heads of ``value_dim``) pass a causal convolution of ``conv_taps`` taps and silu; q and k become unit
    vectors (``unit_eps`` under the root), q times key_dim^-1/2; beta = sigmoid of a projection; the decay is
    g = exp(-exp(A_log) softplus(projection + dt_bias)); per head S <- g S, u = beta (v - S^T k), S <- S + k u^T,
    o = S^T q; o is normed per head, weighted by a weight of size value_dim shared by the heads, gated by silu of a
    projection, and projected out."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    eps: float
    unit_eps: float = 1e-6
    kind: str = "gated_delta"


@dataclass(frozen=True)
class GatedLinearRecurrenceSpec:
    """A recurrent branch beside a gate branch, both ``width`` wide.  y = gelu_tanh(W_y x + b_y); u = conv(W_x x + b_x), a
    causal convolution of ``conv_taps`` taps per channel with a bias; u is cut into ``blocks`` equal parts, and in each
    part two square maps with biases give r = sigmoid(.) and i = sigmoid(.); log f = -``decay_scale`` r softplus(lam);
    per channel s <- f s + sqrt(1 - f^2) i u from s = 0; the output is W_o (s * y)."""
    hidden_size: int
    width: int
    blocks: int
    conv_taps: int
    decay_scale: float = 8.0
    kind: str = "gated_linear_recurrence"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """Matrix memory with exponential input and forget gates, a normaliser and a running maximum that starts at
    zero; gate pre-activations are capped softly at ``gate_cap`` (cap tanh(x / cap)); q is scaled by key_dim^-1/2;
    the read-out is normed per head, weighted over all heads, gated by sigmoid of a projection."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class TimeMixSpec:
    """Linear attention with a decay per token, head and key row, and a bonus for the token's own pair.  Each of the five
    projections (r, k, v, output gate, decay) reads its own blend of the token's input with its predecessor's,
    x + (x' - x) mu.  The decay is exp(-exp(W2 tanh(W1 x_w) + w0)) through a low rank ``decay_rank``.  Per head, with a
    [key_dim, key_dim] state: o = (S + diag(u) k v^T)^T r, then S <- diag(decay) S + k v^T.  Each head's o is divided by
    its root mean square, weighted over all heads, gated by silu of the gate projection, and projected out."""
    hidden_size: int
    num_heads: int
    key_dim: int
    decay_rank: int
    eps: float
    kind: str = "time_mix"


@dataclass(frozen=True)
class StateSpaceSpec:
    """State-space mixer with a scalar decay per token and head.  One projection gives [z | x | B | C | dt]: the gate z
    and the values x (``num_heads`` heads of ``value_dim``), the input and output maps B and C (``groups`` groups of
    ``state_dim``; head h uses group h // (num_heads / groups)) and a step per head.  x, B and C pass a causal
    convolution of ``conv_taps`` taps with a bias, then silu.  dt = softplus(dt + dt_bias); per head
    S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x.  y times silu(z) is normed in ``norm_groups`` equal parts,
    weighted, and projected out."""
    hidden_size: int
    num_heads: int
    value_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    eps: float
    kind: str = "state_space"


@dataclass(frozen=True)
class MixerSumSpec:
    """Several mixers on the same input; the result is the sum of ``scales[i] * mixers[i](x)``.  ``names`` are the
    children's names in parameter names and cache needs."""
    names: Tuple[str, ...]
    mixers: Tuple[Any, ...]
    scales: Tuple[float, ...]
    kind: str = "mixer_sum"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """x += mixer(norm_a(x)) + feed_forward(norm_b(x)), both norms of the same x.  ``feed_forward`` None: the layer
    has none."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    kind: str = "parallel"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down( silu(gate(x)) * up(x) ), dense.  ``interleave``: row layout of the fused gate_up weight:
    0 = all gate rows then all up rows; 8 = blocks of 8 gate rows then their 8 up rows, which lets
    the product's epilogue apply the gate (needs intermediate_size % 8 == 0)."""
    hidden_size: int
    intermediate_size: int
    interleave: int = 0
    kind: str = "swiglu"


@dataclass(frozen=True)
class DenseMLPSpec:
    """down( act(up(x)) ), dense, no gate and no biases.  ``activation``: "relu2" (the square of relu), "gelu_tanh" or
    "silu"."""
    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class ClampedGLUSpec:
    """down( g * sigmoid(alpha g) * (u + 1) ) with g = min(gate(x), limit), u = clamp(up(x), -limit, limit); dense, no
    biases."""
    hidden_size: int
    intermediate_size: int
    limit: float
    alpha: float = 1.702
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class MoESpec:
    """A mixture of ``num_experts`` feed-forwards of one form (``expert``, a dense feed-forward's specification) of which
    every token uses ``top``.  Router scores are a softmax over all experts (float32); with ``groups`` > 1 the experts
    form that many equal groups of neighbours and only those of the ``keep_groups`` groups with the largest best score
    can be chosen; the chosen scores divided by their sum (+ ``renorm_tiny``) weigh the experts' outputs (with
    ``renorm_tiny`` = 0 that is the softmax over the chosen logits alone).  ``router_bias``: a bias per expert is added to
    the logits.  ``expert`` is a ``ClampedGLUSpec`` or a ``SwiGLUSpec`` with rows not woven.  ``shared``: a feed-forward
    that runs for every token and is added, or None.  ``score`` "sigmoid": every expert's score is the logistic of its own
    logit instead of a softmax over all.  ``group_top`` 2: a group is ranked by the sum of its two largest scores instead of
    its largest.  ``weight_scale``: a factor on the weights after they were divided by their sum."""
    hidden_size: int
    num_experts: int
    top: int
    expert: Any
    groups: int = 1
    keep_groups: int = 1
    shared: Any = None
    renorm_tiny: float = 1e-20
    router_bias: bool = False
    kind: str = "moe"
    score: str = "softmax"
    group_top: int = 1
    weight_scale: float = 1.0


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x += post_a(mixer(pre_a(x))); x += post_b(feed_forward(pre_b(x))): a norm before and after each sublayer.
    ``feed_forward`` None: the layer has none (and no norms for it)."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    mixer_post_norm: Any
    feed_forward_norm: Any = None
    feed_forward_post_norm: Any = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class HyperBlockSpec:
    """A pre-norm layer over ``streams`` residual streams x_1 .. x_S instead of one.  Each sublayer has a read vector
    a [S], a write vector b [S] and a mixing matrix m [S, S] (indexed [from, to]): it runs on norm(sum_s a[s] x_s),
    and then x_t <- sum_s m[s, t] x_s + b[t] y for all t at once.  ``feed_forward`` None: the layer has none.
    ``learned`` False: a, b and m are not parameters but all one, which with one stream is the plain residual sum
    x <- x + y."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    streams: int
    learned: bool = True
    kind: str = "hyper"


@dataclass(frozen=True)
class BlockSpec:
    """The arrangement of one layer: x += m * mixer(norm(x)); x += m * feed_forward(norm(x)), with m =
    ``residual_scale``.  ``feed_forward`` None: the layer has none (and no norm for it)."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    kind: str = "prenorm"
    residual_scale: float = 1.0
    float_outputs: bool = False           # the sublayers may hand back float32 on the bfloat16 path (the adds then run in
                                          # the kernel that takes either type)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` None: the run owns a cache of its own; an index: the run
    reads the cache that the schedule entry with that index wrote, and writes none."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class DecoderSpec:
    vocab_size: int
    hidden_size: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_embeddings: bool
    embedding_norm: Any = None            # a norm applied to the embedded tokens before the first layer
    logit_softcap: Optional[float] = None  # logits <- cap * tanh(logits / cap)
    embedding_scale: float = 1.0          # the embedded tokens are multiplied by this (the output head is not)
    # (buckets, mul_prev, mul_cur): a table ``embed_pairs`` [buckets + 1, hidden] adds the row
    # (previous token * mul_prev + token * mul_cur) mod buckets to an embedded token (after the scale), and its last row
    # to a sequence's first token; a request's last token is then part of its state
    embedding_pairs: Optional[Tuple[int, int, int]] = None
    streams: Optional[int] = None         # None: one residual stream [T, hidden].  n: a token has n streams
                                          # ([T, n, hidden]; every block must take them), all start as the embedded
                                          # token and their sum goes to the final norm

    @staticmethod
    def in_order(n_layers: int) -> Tuple[ScheduleEntry, ...]:
        return tuple(ScheduleEntry(i) for i in range(n_layers))

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, there are {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns none")
