"""Descriptions of a model as data: which parts, of which sizes, in which order.

An architecture turns its typed configuration into one :class:`ModelSpec`.
Nothing below names an architecture: every size and constant is a field, every
layer has its own list of sub-layers (a mixer or a feed-forward with its norms each), and the order in which
layers run is the ``schedule`` list, which may name a layer twice or let two
entries use one cache.

A part's description is any frozen dataclass with a ``kind`` string; the
``kind`` selects the implementation in :mod:`inferrs_b200.parts.registry`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor that a part expects in the weight files.

    ``init`` tells the random-weights mode how to fill it: ``"normal"`` is
    N(0, 0.02), ``"norm"`` is 1 + U(-0.1, 0.1), ``"uniform:c:r"`` is c + U(-r, r),
    ``"identity:r"`` (a square matrix) is the identity plus U(-r, r).  ``optional``
    tensors may be absent; the part says what it does then.
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class NormSpec:
    """x / sqrt(mean(x^2) + eps) * weight.  ``groups`` > 1: the row is cut into that many equal consecutive parts
    and each part is divided by its own root mean square.  ``weight`` None (where a part allows it: the per-head
    norms of attention): the division alone.  ``kind="layer_norm"``: (x - mean) / sqrt(variance + eps) * weight, the
    variance being the mean of the squared deviations from the mean; no bias."""

    size: int
    eps: float
    weight: Optional[str]
    kind: str = "rms"
    groups: int = 1


@dataclass(frozen=True)
class PositionSpec:
    """Rotation of the first ``rot_dim`` elements of each head by position.

    ``kind="rotary_split_half"`` pairs element ``i`` with ``i + rot_dim/2``;
    ``kind="rotary_interleaved"`` pairs element ``2i`` with ``2i + 1``;
    ``kind="none"`` leaves heads as they are.  ``kind="rotary_scaled"`` pairs like ``rotary_split_half`` and stretches
    the slow pairs for contexts longer than the ``original`` one (``scaling`` = (factor, original, fast, slow): with
    turns(t) = rot_dim ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turns(fast)), 0),
    hi = min(ceil(turns(slow)), rot_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1).
    """

    kind: str = "rotary_split_half"
    rot_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache of keys and values.

    ``window``: a query at position i sees keys j with i - window < j <= i;
    ``None`` means all keys j <= i.  ``chunk``: a query sees only the keys of its own chunk of that many positions,
    counted from position 0 of the sequence (floor(i / chunk) = floor(j / chunk)).  ``own_kv=False`` describes a
    layer that has no key/value projections and reads the cache that another schedule
    entry writes.  ``value_dim``: the size of a value head where it differs from ``head_dim``.
    ``norm_after_rotation``: the per-head norms of queries and keys come after the rotation instead of before it.
    ``q_bias`` / ``k_bias`` / ``v_bias`` / ``o_bias``: vectors added to the projections' results.
    ``distance_bias`` = (r1, r2), two tensors [n_heads]: r1_h ln(1 + r2_h (i - j)) is taken off head h's scaled score
    of query i against key j.  ``head_mix`` [n_heads, n_heads]: after that the heads' scores are mixed,
    score_h <- sum_g mix[h, g] score_g, before mask and softmax (every head still reads the values of its own group).

    ``distance_slopes`` (one constant per head): slope_h (i - j) is taken off head h's scaled score.
    ``head_scale`` [n_heads]: head h's scaled score is multiplied by a learned number.
    ``sink`` [n_heads]: every row's softmax gets one more term, exp(sink_h), in its denominator only; no key or value
    belongs to it, and ``scale``, ``head_scale`` and the distance terms leave it alone.
    ``qkv_conv`` = (q, k, v tensor names, each [channels, ``conv_taps``]): a causal convolution per channel directly
    behind each projection (the last tap weighs the token itself, zeros before the start, no bias, no activation);
    the last conv_taps - 1 projected rows of a request belong to its state.
    ``norm_whole``: ``q_norm`` / ``k_norm`` are taken over the whole projection, all heads at once (their ``size`` is
    n_heads * head_dim and n_kv_heads * head_dim), instead of per head.
    ``gate_proj`` [n_heads * value_dim, width]: the heads side by side are multiplied by sigmoid(gate(x)) before
    ``o_proj``.
    ``value_publish``: the layer's values of the step's rows, as they are cached, are kept under this name for later
    layers of the same step.  ``value_blend`` = (name, weight tensor of one number): v <- (1 - w) v + w v_name with
    the values that an earlier layer published under that name, before v is cached.  ``unused``: tensors that the
    weight files hold for this layer and that nothing reads.
    """

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    q_proj: str
    o_proj: str
    k_proj: Optional[str] = None
    v_proj: Optional[str] = None
    q_norm: Optional[NormSpec] = None
    k_norm: Optional[NormSpec] = None
    window: Optional[int] = None
    own_kv: bool = True
    kind: str = "attention"
    value_dim: Optional[int] = None
    chunk: Optional[int] = None
    norm_after_rotation: bool = False
    q_bias: Optional[str] = None
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    o_bias: Optional[str] = None
    distance_bias: Optional[Tuple[str, str]] = None
    head_mix: Optional[str] = None
    distance_slopes: Optional[Tuple[float, ...]] = None
    head_scale: Optional[str] = None
    sink: Optional[str] = None
    qkv_conv: Optional[Tuple[str, str, str]] = None
    conv_taps: int = 0
    norm_whole: bool = False
    gate_proj: Optional[str] = None
    value_publish: Optional[str] = None
    value_blend: Optional[Tuple[str, str]] = None
    unused: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()


@dataclass(frozen=True)
class GatedDenseSpec:
    """down( act(gate(x)) * up(x) ).  ``activation="clamped_swish"``: with g = min(gate(x), limit) and
    u = clamp(up(x), -limit, limit) the inner rows are g sigmoid(slope g) (u + 1).  ``activation="gelu_tanh"``:
    act(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))."""

    width: int
    inner: int
    gate_proj: str
    up_proj: str
    down_proj: str
    activation: str = "silu"
    kind: str = "gated_dense"
    limit: Optional[float] = None
    slope: float = 1.702


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of small gated feed-forwards.  Router logits z = router(x) + router_bias in float32; the ``top``
    experts with the largest logits are chosen and weighed by the softmax over the chosen logits alone; the output is
    the weighted sum of down_e( silu(gate_e(x)) * up_e(x) ) over the chosen.  ``experts`` names every expert's
    (gate, up, down) tensors.  ``shared`` (optional, (gate, up, down, gate vector) with ``shared_inner``): an expert
    that every token uses; its output is added times sigmoid(gate_vector . x).
    ``scoring="sigmoid_share"``: the scores are s = sigmoid(z), the ``top`` largest scores are chosen, and a chosen
    expert weighs s_e / (sum of the chosen scores + 1e-20).  ``scoring="softmax_share"``: the same with the scores
    s = softmax(z) over all experts.  ``route_scale`` multiplies the routed experts' weights.
    ``activation="clamped_swish"`` (with ``limit`` and ``slope``): an expert is down_e( g sigmoid(slope g) (u + 1) )
    with g = min(gate_e(x), limit) and u = clamp(up_e(x), -limit, limit)."""

    width: int
    inner: int
    top: int
    router: str
    router_bias: Optional[str]
    experts: Tuple[Tuple[str, str, str], ...]
    shared: Optional[Tuple[str, str, str, str]] = None
    shared_inner: int = 0
    kind: str = "routed_experts"
    scoring: str = "softmax_of_chosen"
    route_scale: float = 1.0
    activation: str = "silu"
    limit: Optional[float] = None
    slope: float = 1.702


@dataclass(frozen=True)
class FixedDecayScanSpec:
    """Retention: linear attention whose state fades by a fixed factor per head; the scores go through no softmax and no normaliser.  Per head a
    matrix state S [key_dim, value_dim], S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; q and k are rotated by
    position (``position``), k is then multiplied by key_dim^(-1/2) (``key_scale`` if given); each head's o is divided
    by its root mean square (no weight); the heads times silu(gate(x)) go through ``o_proj``.
    ``input_activation="silu"``: q, k and v go through silu as they leave their projections (such heads are not
    rotated).  ``norm_heads_together``: the heads' o side by side are divided by one root mean square over all of
    them.  ``out_norm`` [n_heads * value_dim]: a weight on the normed o.  ``gate_activation``: "silu" or "sigmoid"."""

    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    eps: float
    position: PositionSpec
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    kind: str = "fixed_decay_scan"
    input_activation: Optional[str] = None
    key_scale: Optional[float] = None
    norm_heads_together: bool = False
    out_norm: Optional[str] = None
    gate_activation: str = "silu"


@dataclass(frozen=True)
class GatedDeltaScanSpec:
    """The gated delta rule.  q and k [n_kv_heads, key_dim] and v [n_heads, value_dim] leave their projections through
    a causal convolution per channel over the last ``taps`` inputs (``*_conv`` [channels, taps], the last tap weighing
    the token itself, no bias, zeros before the start) and silu; q and k are then made unit vectors per head,
    x / sqrt(sum(x^2) + unit_eps), and q is multiplied by key_dim^(-1/2).  Per head (head h reads q/k head
    h / (n_heads / n_kv_heads)) a state S [key_dim, value_dim] with beta = sigmoid(beta_proj(x)) and
    fade = exp(-exp(a_log_h) softplus(a_proj(x) + dt_bias_h)):
    S <- fade S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q (the read-out sees the token's own write).
    Each head's o is divided by its root mean square (``eps``), multiplied by ``out_norm`` [value_dim] (one weight for
    all heads) and by silu(gate(x)), and goes through ``o_proj``.  The convolutions' last taps - 1 inputs belong to
    the per-request state."""

    width: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    taps: int
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    q_conv: str
    k_conv: str
    v_conv: str
    beta_proj: str
    a_proj: str
    a_log: str
    dt_bias: str
    gate_proj: str
    out_norm: str
    o_proj: str
    unit_eps: float = 1e-6
    kind: str = "gated_delta_scan"


@dataclass(frozen=True)
class MixerSumSpec:
    """Two mixers side by side on the same input: ``left_scale`` * left(x) + ``right_scale`` * right(x).  The layer's
    schedule entry names one cache id; at most one of the two keeps pages of keys and values and at most one a
    per-request state (one of each is fine: they share the id)."""

    left: Any
    right: Any
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "mixer_sum"


@dataclass(frozen=True)
class StateSpaceScanSpec:
    """The state-space mixer of Mamba-2.  The columns of ``in_proj``'s output are, in order: the gate z (inner), x
    (inner), B (groups * state), C (groups * state) and dt (n_heads), with inner = n_heads * value_dim.  x, B and C
    go through a causal convolution per channel over the last ``taps`` inputs (``conv`` [channels, taps], the last tap
    weighing the token itself, plus ``conv_bias``) and silu; dt = softplus(dt + dt_bias).  Per head (head h reads
    group h / (n_heads / groups) of B and C) a state S [state, value_dim]:
    S_t = exp(-exp(a_log_h) dt) S_{t-1} + dt B_t x_t^T, y_t = S_t^T C_t + skip_h x_t.  y silu(z) is divided by its
    root mean square in ``norm_groups`` equal parts (gated first, normed second), multiplied by ``out_norm`` and goes
    through ``o_proj``.  The convolution's last taps - 1 inputs belong to the per-request state."""

    width: int
    n_heads: int
    value_dim: int
    state: int
    groups: int
    taps: int
    norm_groups: int
    eps: float
    in_proj: str
    conv: str
    conv_bias: str
    dt_bias: str
    a_log: str
    skip: str
    out_norm: str
    o_proj: str
    kind: str = "state_space_scan"


@dataclass(frozen=True)
class PolyNormDenseSpec:
    """down( act(up(x)) ) with act(z) = a U(z) + b U(z^2) + c U(z^3) + e, powers element by element, U the division
    of a row by its root mean square (``eps`` inside the root); ``coef`` names the tensor (a, b, c, e)."""

    width: int
    inner: int
    up_proj: str
    down_proj: str
    coef: str
    eps: float
    kind: str = "poly_norm_dense"


@dataclass(frozen=True)
class ChannelDecayScanSpec:
    """Gated linear attention: per head a matrix state S [key_dim, value_dim] with a decay per key channel,
    S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, q scaled by key_dim^(-1/2),
    a_t = sigmoid(up(down(x)) + bias)^(1/tau).  Each head's o is divided by its root mean square and multiplied by
    ``out_norm`` [value_dim] (one weight for all heads); the heads times silu(gate(x)) go through ``o_proj``."""

    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    decay_down: str
    decay_up: str
    decay_bias: str
    out_norm: str
    kind: str = "channel_decay_scan"


@dataclass(frozen=True)
class ForgetWriteScanSpec:
    """HGRN2: a linear recurrence whose key is the complement of its forget gate.  Per head a matrix state S
    [key_dim, value_dim]: f = l + (1 - l) sigmoid(f_proj(x) + f_bias) per key channel with a learned lower bound l
    (``lower`` [n_heads * key_dim]); S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t with
    q = silu(q_proj(x)) and v = v_proj(x); there is no key and no other scale.  Each head's o is divided by its root
    mean square and multiplied by ``out_norm`` [value_dim] (one weight for all heads); the heads go through
    ``o_proj``.  The gate, its complement and the state are float32."""

    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    eps: float
    q_proj: str
    f_proj: str
    f_bias: str
    lower: str
    v_proj: str
    out_norm: str
    o_proj: str
    kind: str = "forget_write_scan"


@dataclass(frozen=True)
class ScalarGateScanSpec:
    """The matrix memory of xLSTM: per head a state S [key_dim, value_dim], a vector n and a running maximum m, moved
    by a log input gate i = cap tanh((W_i x + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f x + b_f) /
    cap)): m' = max(f + m, i), S' = exp(f + m - m') S + exp(i - m') k v^T (n likewise), o = S'^T q / (max(|n' . q|,
    exp(-m')) + 1e-6), q scaled by key_dim^(-1/2).  Each head's o is divided by its root mean square; the heads times
    ``out_norm`` [n_heads * value_dim] times sigmoid(gate(x)) go through ``o_proj``."""

    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    i_proj: str
    i_bias: str
    f_proj: str
    f_bias: str
    out_norm: str
    kind: str = "scalar_gate_scan"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are made per head from one cached latent per token, without positions.

    c_q = rmsnorm(dq(x)), q = uq(c_q) [n_heads, key_dim]; c = rmsnorm(dkv(x)) [kv_rank] is what the cache holds;
    k_h = uk_h c, v_h = uv_h c [value_dim]; scores (q . k) * scale over j <= i (``window``: i - window < j), softmax;
    the heads times sigmoid(gate(x)) go through ``o_proj``.  ``own_kv=False``: the layer has no ``dkv`` and reads
    the latents that another schedule entry writes."""

    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    eps: float
    dq_proj: str
    dq_norm: str
    uq_proj: str
    uk_proj: str
    uv_proj: str
    gate_proj: str
    o_proj: str
    dkv_proj: Optional[str] = None
    dkv_norm: Optional[str] = None
    window: Optional[int] = None
    own_kv: bool = True
    kind: str = "latent_attention"


@dataclass(frozen=True)
class StreamConnectionSpec:
    """How a sub-layer hangs on a residual that is ``streams`` copies wide (hyper-connections): it reads
    u = sum_s read[s] x_s, and its output y comes back as x_t <- sum_s mix[s, t] x_s + gain[t] y (all t at once from
    the old streams).  The three fields name the tensors [streams], [streams], [streams, streams]."""

    streams: int
    read: str
    gain: str
    mix: str


@dataclass(frozen=True)
class InputConvSpec:
    """A short convolution over time between a sub-layer's norm and its part.  With h the norm's output [rows, width],
    the part is handed h + c(h), where c works on every channel by itself:
    c(h)_t = sum_{j < taps} weight[:, j] * h_(t - (taps - 1 - j)); rows that would lie ahead of a request's first token
    count as zero.  ``weight`` names the tensor [width, taps] (the last column multiplies the row itself; no bias).  A
    request's state keeps the taps - 1 most recent rows of h, so that a later step can go on where this one ended."""

    width: int
    taps: int
    weight: str


@dataclass(frozen=True)
class ResidualGateSpec:
    """A sub-layer's result is multiplied element by element by sigmoid(weight h + bias) before it joins the stream,
    h being what the sub-layer itself reads (the norm's output).  ``weight`` [width, width], ``bias`` [width]."""

    weight: str
    bias: str


@dataclass(frozen=True)
class SubLayerSpec:
    """One sub-layer of a block: a part with what stands before and after it.

    ``category`` says which registry the part's ``kind`` is looked up in: ``"mixer"`` (it gets the
    layer's cache) or ``"feed_forward"``.  ``norm`` is applied to the residual stream before the part
    (``None``: the part reads the stream as it is); ``post_norm`` to the part's output before it is
    added to the stream (``None``: it is added as it is).
    """

    part: Any
    category: str
    norm: Optional[Any] = None
    post_norm: Optional[Any] = None
    # for arrangements whose sub-layers hang on the residual in a way of their own (StreamConnectionSpec,
    # ResidualGateSpec)
    connection: Optional[Any] = None
    # for the arrangement that norms after the sum: the norm of the stream itself once the part's output is in it
    sum_norm: Optional[Any] = None
    # a short convolution over time on what the part reads (InputConvSpec), for arrangements that apply it
    input_conv: Optional[Any] = None


@dataclass(frozen=True)
class LayerSpec:
    """One block: its sub-layers, in order, and how they are arranged around the residual stream.

    ``arrangement="sequential"``: for every sub-layer in turn, x += post_norm(part(norm(x))).  A
    pre-norm block of a mixer and a feed-forward is two sub-layers with a ``norm`` each
    (:func:`pre_norm_layer`); a block with four norms gives both a ``post_norm`` too; a block of a
    mixer alone has one sub-layer.

    ``arrangement="norm_after_sum"``: for every sub-layer in turn, x <- sum_norm(residual_scale * x + part(x)): the
    parts read the stream itself, and the stream itself is normalised (``part`` None: the sum is residual_scale * x).

    ``arrangement="gated_residual"``: for every sub-layer in turn, h = norm(x), x += sigmoid(W h + b) * part(h), with
    W and b from the sub-layer's ``connection`` (a :class:`ResidualGateSpec`).
    """

    sublayers: Tuple[SubLayerSpec, ...]
    arrangement: str = "sequential"
    residual_scale: float = 1.0

    def parts_of(self, category: str) -> Tuple[Any, ...]:
        return tuple(s.part for s in self.sublayers if s.category == category)

    @property
    def mixer(self) -> Any:
        """The layer's mixer description (the first, if it has several; None if it has none)."""
        return next(iter(self.parts_of("mixer")), None)

    @property
    def ffn(self) -> Any:
        """The layer's feed-forward description (the first, if it has several; None if it has none)."""
        return next(iter(self.parts_of("feed_forward")), None)

    def with_part(self, category: str, part: Any, index: int = 0) -> "LayerSpec":
        """A copy in which the ``index``-th sub-layer of ``category`` has another part."""
        seen, subs = 0, []
        for s in self.sublayers:
            if s.category == category:
                if seen == index:
                    s = SubLayerSpec(part=part, category=category, norm=s.norm, post_norm=s.post_norm,
                                     connection=s.connection, sum_norm=s.sum_norm, input_conv=s.input_conv)
                seen += 1
            subs.append(s)
        if seen <= index:
            raise ValueError(f"the layer has {seen} sub-layers of category '{category}', none with index {index}")
        return LayerSpec(sublayers=tuple(subs), arrangement=self.arrangement, residual_scale=self.residual_scale)


def pre_norm_layer(mixer_norm: Any, mixer: Any, ffn_norm: Any, ffn: Any) -> LayerSpec:
    """x += mixer(norm(x)); x += feed_forward(norm(x))."""
    return LayerSpec(sublayers=(SubLayerSpec(part=mixer, category="mixer", norm=mixer_norm),
                                SubLayerSpec(part=ffn, category="feed_forward", norm=ffn_norm)))


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer`` with cache ``cache``.

    ``cache`` numbers the caches (and fixed-size states) of the model.  Two
    entries with the same ``layer`` share weights; two entries with the same
    ``cache`` share keys and values (exactly one of them writes).
    """

    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    width: int
    embedding: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    lm_head: str
    # True: the head tensor may be absent, the embedding table is used then.
    lm_head_optional: bool
    max_positions: int
    # embedding rows are multiplied by this as they are gathered (None: not at all)
    embedding_scale: Optional[float] = None
    # a norm on the embedding rows before the first layer (None: none)
    embedding_norm: Optional[Any] = None
    # logits are multiplied by logit_scale and then squashed to cap * tanh(x / cap) (None: neither)
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    # a learned vector per position [max_positions, width] that is added to the embedding (None: no such table)
    position_table: Optional[str] = None
    # the residual is this many streams wide, [rows, streams, width], all equal to the embedding at the start and
    # summed before the last norm (None: the plain residual [rows, width])
    streams: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ""
    extra: Tuple[Tuple[str, Any], ...] = field(default_factory=tuple)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))
