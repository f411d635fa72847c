"""Typed descriptions of a model: what each layer is made of, and in which
order layers run.

A configuration class of an architecture turns its ``config.json`` into a
``ModelSpec``.  Everything below the specs (parts, cache, engine) reads sizes
and constants from here and from nowhere else; none of it knows which
architecture it serves.

The reference resolves the same facts per layer at load time into its
``Layer`` records (crates/nncpu/src/model/mod.rs:103-194): head counts, window,
which cache a layer reads, whether it keeps recurrent state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over a vector of ``size`` lanes, weights at ``name + suffix``.  ``offset`` is added to
    the stored weight before it multiplies (1.0 for weights that are stored around zero).  ``kind`` "rmsnorm":
    x / sqrt(mean(x^2) + eps) * w.  ``kind`` "layernorm": (x - mean) / sqrt(var + eps) * w + b with var the mean of the
    squared deviations and the bias b at ``name + suffix + bias_suffix``."""
    kind: str
    size: int
    eps: float
    name: str  # tensor name prefix, e.g. "model.layers.0.input_layernorm"
    suffix: str = ".weight"
    offset: float = 0.0
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer.  ``kind`` "rope_neox": rotate the pairs
    (i, i + rotary_dim/2) of the first ``rotary_dim`` lanes of a head by
    position * theta^(-2i/rotary_dim).  ``kind`` "rope_pairs": the same angles on the pairs (2i, 2i + 1)."""
    kind: str
    theta: float
    rotary_dim: int
    position_scale: float = 1.0
    # Frequencies rescaled between two wavelengths (``scaling_factor`` > 0): with n(t) = rotary_dim * ln(original /
    # (2 pi t)) / (2 ln theta), lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), rotary_dim - 1) and
    # ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i),
    # and cos and sin are multiplied by 0.1 * ln(factor) + 1.
    scaling_factor: float = 0.0
    scaling_original: float = 0.0
    scaling_fast: float = 0.0
    scaling_slow: float = 0.0


@dataclass(frozen=True)
class MixerSpec:
    """The part of a block that looks at other positions.  Subclasses add
    their sizes; ``kind`` picks the implementation from the mixer registry and
    ``name`` is the prefix of its tensors."""
    kind: str
    name: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias_optional: bool = False  # accept "<name>.o_proj.bias" when the file has it
    scale: float = 0.0               # multiplies q.k after the dot product
    window: int = 0                  # 0: every earlier key; n: the last n keys up to the query
    qk_norm: Optional[NormSpec] = None   # per-head norm of q and k (names end in q_norm / k_norm)
    position: Optional[PositionSpec] = None
    v_head_dim: int = 0              # lanes of a value head (and of a head's output); 0: head_dim
    slope_base: float = 0.0          # b != 0: head h takes 2^(-b (h + 1) / n_heads) * (i - j) off its scaled scores
    q_temp_coef: float = 0.0         # c != 0: the query at position p is multiplied by
    q_temp_every: int = 1            # 1 + c * ln(floor((p + 1) / every) + 1)
    tensor_names: str = "proj"       # "proj": <name>.q_proj.weight / .bias ...; "short": <name>.q, <name>.q.b, ... <name>.o
    chunk: int = 0                   # n: positions are cut into blocks of n from position 0 of the sequence, and a
                                     # query sees the keys of its own block up to itself (not together with window)
    out_bias: bool = False           # the output projection has a bias (required, unlike out_bias_optional)
    values_are_keys: bool = False    # no value projection: a position's value is its key as projected, before the
                                     # per-head norm and the rotation
    sink: bool = False               # a learned logit per head ("<name>.sink") whose exponential joins the softmax's
                                     # denominator: it has no key and no value, is not scaled, and counts once
    out_gate: bool = False           # the concatenated heads are multiplied, lane by lane, by sigmoid(W_g h)
                                     # ("<name>.g", n_heads * v_head_dim rows) before the output projection


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Attention whose keys and values are products of one latent vector per position: c = rmsnorm(W_dkv h) of
    ``latent_dim`` lanes is all that is kept; head a has k = W_uk[a] c (``head_dim`` lanes) and v = W_uv[a] c
    (``v_head_dim`` lanes).  Causal; scores times ``scale``.  With ``head_gate`` every head's
    output is multiplied by the sigmoid of one more projection of h (one logit per head).

    ``rot_dim`` R > 0: a head's query has R more lanes after its ``head_dim`` unrotated ones, W_dkv has R more rows
    after the latent's (not normed), and those R lanes, rotated by ``position``, are one key part that all heads
    share: score = (q_unrotated . k_unrotated + q_rotated . k_rotated) * scale; the latent and the rotated key part
    are what is kept.  ``q_rank`` > 0: queries go through a latent of their own, q = W_uq rmsnorm(W_dq h).
    ``sink``: as in ``AttentionSpec``.  A layer that reads another layer's cache has no W_dkv."""
    hidden_size: int = 0
    n_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    latent_dim: int = 0
    scale: float = 0.0
    eps: float = 1e-6
    head_gate: bool = False
    rot_dim: int = 0
    position: Optional[PositionSpec] = None
    q_rank: int = 0
    sink: bool = False


@dataclass(frozen=True)
class RetentionSpec(MixerSpec):
    """Retention, a recurrent mixer: linear attention with one fixed decay per head and neither softmax nor
    denominator.  q, k (``n_heads`` x ``key_dim``) and v (``n_heads`` x ``value_dim``) are projections without biases;
    q and k are rotated by ``position`` (optional), k is then multiplied by key_dim^-1/2; per head
    S_t = decays[h] S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  Every head's o is divided by its root mean square (``eps``,
    no weight); the concatenated heads are multiplied by silu(W_g h) and projected back (``<name>.q / .k / .v / .g /
    .o``).  The state is 32-bit."""
    hidden_size: int = 0
    n_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    decays: Tuple[float, ...] = ()
    position: Optional[PositionSpec] = None
    eps: float = 1e-6


@dataclass(frozen=True)
class MixerPairSpec(MixerSpec):
    """Two mixers side by side that read the same input: the result is ``weight`` times the sum of their outputs, each
    first RMS-normed over the model width (``eps``) with a plain weight of its own, ``<name>.<left|right>.out``; the
    mixers' own tensors lie under ``<name>.left`` and ``<name>.right``."""
    hidden_size: int = 0
    left: Optional[MixerSpec] = None
    right: Optional[MixerSpec] = None
    eps: float = 1e-6
    weight: float = 0.5


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """The gated delta rule, a recurrent mixer: per head a state S of ``key_dim`` x ``value_dim`` 32-bit numbers.
    q and k have ``n_kv_heads`` heads (head h of ``n_heads`` uses q/k head h // (n_heads / n_kv_heads)), v has
    ``n_heads``; each passes a causal convolution of ``conv`` taps per channel and SiLU; q and k become unit vectors
    (x / sqrt(sum x^2 + 1e-6); q also times key_dim^-1/2).  Per token and head: beta = sigmoid(W_b h),
    g = exp(-exp(A_log) softplus(W_a h + dt_bias)); S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    The heads' outputs are RMS-normed (``eps``, one weight of ``value_dim`` lanes), gated by silu(W_g h) and projected
    back.  The last ``conv`` - 1 inputs of the convolutions are state too.

    ``channel_decay``: one decay per head AND key channel, acting on the rows of S,
    g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias)) laid out heads x key_dim (``<name>.a1`` [r, hidden],
    ``.a2`` [H key_dim, r], ``.dt_bias`` [H key_dim]; the rank r is what the file's tensors have), and the output gate is
    sigmoid(W_g2 (W_g1 h)) laid out heads x value_dim (``.g1``, ``.g2``) in place of silu(W_g h)."""
    hidden_size: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    conv: int = 0
    eps: float = 1e-6
    channel_decay: bool = False
    decay_rank: int = 0     # 0: what the file's tensors have
    gate_rank: int = 0


@dataclass(frozen=True)
class GatedLinearAttentionSpec(MixerSpec):
    """A recurrent mixer: per head a state of ``key_dim`` x ``value_dim`` numbers that decays per key channel by
    sigmoid(z)^(1/tau), z from a low-rank projection (``gate_rank``) with a bias; the heads' outputs are
    RMS-normed (``eps``), gated by silu of a projection and projected back."""
    hidden_size: int = 0
    n_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    gate_rank: int = 0
    tau: float = 1.0
    eps: float = 1e-6


@dataclass(frozen=True)
class FeedForwardSpec:
    """The part of a block that works on each position alone."""
    kind: str
    name: str


@dataclass(frozen=True)
class GatedMlpSpec(FeedForwardSpec):
    """down(act(gate(x), up(x))).  ``activation`` "silu": silu(g) u; "gelu_tanh": the tanh form of GELU of g, times u;
    "swish_clamp": with g' = min(g, limit) and u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1)."""
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    limit: float = 0.0
    tensor_names: str = "proj"       # "proj": <name>.gate_proj.weight ...; "short": <name>.gate, <name>.up, <name>.down


@dataclass(frozen=True)
class RoutedExpertsSpec(FeedForwardSpec):
    """``n_experts`` small gated feed-forwards (``<name>.e<i>.gate / .up / .down``) of which every token uses the
    ``top`` with the largest router logits (``<name>.router`` with the bias ``<name>.router.b``, in 32-bit), weighted
    by the softmax over the chosen logits alone; plus an optional ``shared`` gated feed-forward that every token runs.

    ``scores`` "all": the scores are the softmax over ALL experts' logits; the ``top`` experts with the largest scores
    are chosen, and their weights are their scores divided by the sum of the chosen scores (+ 1e-20), times
    ``weight_scale``.  With ``n_groups`` > 1 the experts form that many equal groups of neighbours, a group's score is
    its largest score, and only experts of the ``keep_groups`` best groups can be chosen.  ``router_bias`` False: the
    router has no bias tensor.  ``out_scale`` multiplies what the part adds to the stream."""
    hidden_size: int = 0
    intermediate_size: int = 0
    n_experts: int = 0
    top: int = 0
    activation: str = "swish_clamp"
    limit: float = 0.0
    shared: Optional[GatedMlpSpec] = None
    scores: str = "chosen"
    n_groups: int = 1
    keep_groups: int = 1
    weight_scale: float = 1.0
    router_bias: bool = True
    out_scale: float = 1.0


@dataclass(frozen=True)
class DenseMlpSpec(FeedForwardSpec):
    """down(act(up(x))) with biases on both products (``bias`` False: without); ``activation`` "xielu" has two learned
    numbers at ``<name>.act``, "relu2" is the square of relu."""
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "xielu"
    bias: bool = True


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, added to the stream at the end of a layer: with e the lanes
    [``col``, ``col`` + ``dim``) of row ``token`` of the table ``table`` [vocab, ``table_width``],
    y = W_proj (gelu_tanh(W_gate x) * e) and x <- x + mult * y / sqrt(mean(y^2) + eps) * w
    (``<name>.gate`` [dim, hidden], ``.proj`` [hidden, dim], ``.norm`` [hidden]; mult is the block's ``residual_mult``)."""
    name: str
    table: str
    table_width: int
    col: int
    dim: int
    hidden_size: int
    vocab_size: int
    eps: float = 1e-6


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and their arrangement.  ``kind`` "prenorm":
    x += mixer(norm1(x)); x += feed_forward(norm2(x)).  ``kind`` "sandwich" norms each sublayer's output too:
    x += norm1_post(mixer(norm1(x))); x += norm2_post(feed_forward(norm2(x))), and a layer without a
    feed-forward (``feed_forward`` None) has the first sublayer only.  ``kind`` "parallel": both sublayers read the
    stream as it enters the layer, x += mixer(norm1(x)) + feed_forward(norm2(x)); without a feed-forward norm2 is not used (its tensor is optional);
    a "parallel" layer with a feed-forward and ``norm2`` None has one norm, whose output both sublayers read.
    ``residual_mult`` m ("prenorm"): x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x)), and a "prenorm" layer
    may go without a feed-forward.  ``side`` ("prenorm"): a per-layer token input after the feed-forward."""
    kind: str
    norm1: NormSpec
    mixer: MixerSpec
    norm2: Optional[NormSpec] = None
    feed_forward: Optional[FeedForwardSpec] = None
    norm1_post: Optional[NormSpec] = None
    norm2_post: Optional[NormSpec] = None
    residual_mult: float = 1.0
    side: Optional[TokenSideSpec] = None


@dataclass(frozen=True)
class StreamInjection:
    """What is added to the residual stream right before a schedule entry runs: with ``embedding`` the stream as the
    embedding left it (before the first layer), and row ``row`` of the tensor ``table`` [``n_rows``, hidden].
    ``mix`` (a tensor [hidden, 2 hidden]): first the stream becomes W_mix [x; x0], x0 the stream as the embedding left
    it (x's columns first); the table's row is added after that."""
    embedding: bool = False
    table: Optional[str] = None
    n_rows: int = 0
    row: int = 0
    mix: Optional[str] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` and may
    appear in several entries (the layer then runs again with the same
    weights and a cache of its own).  ``cache_of`` names an earlier entry
    whose keys and values this run reads instead of keeping its own.  ``inject``: what the stream receives
    before this run (a schedule that repeats a range of layers marks the start of each pass this way)."""
    layer: int
    cache_of: Optional[int] = None
    inject: Optional[StreamInjection] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    name: str          # tensor name of the table, without the suffix
    vocab_size: int
    hidden_size: int
    scale: float = 1.0
    suffix: str = ".weight"
    positions: Optional[str] = None   # tensor name of a table of learned position vectors [n_positions, hidden],
    n_positions: int = 0              # added (unscaled) to the embedding rows; sequences cannot outgrow it
    # A hashed embedding of the pair (previous token, token), added to the embedding row: row
    # (previous * pair_mul_prev + token * pair_mul_cur) mod pair_buckets of the tensor ``pair_table``
    # [pair_buckets + 1, hidden]; a sequence's first token takes the last row.  The previous token is per-sequence state.
    pair_table: Optional[str] = None
    pair_buckets: int = 0
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0


@dataclass(frozen=True)
class OutputSpec:
    """Final norm and vocabulary projection.  ``tied`` uses the embedding
    table as the output matrix."""
    norm: NormSpec
    name: str          # tensor name of the output matrix, without the suffix
    tied: bool
    vocab_size: int
    hidden_size: int
    suffix: str = ".weight"
    softcap: float = 0.0   # c > 0: logits <- c * tanh(logits / c)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    output: OutputSpec
    stop_token_ids: Tuple[int, ...] = field(default_factory=tuple)
