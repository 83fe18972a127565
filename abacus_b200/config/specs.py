"""Descriptions of the parts a model is put together from.

A spec is plain data: the sizes and constants one part needs, nothing about the
model it sits in. An architecture's configuration turns its config.json into a
`ModelSpec`: one `BlockSpec` per layer (so layers may differ), and a schedule,
the order in which layers run.

Every spec class carries a `kind`; the part registries (abacus_b200.parts) map
a kind to the class that implements it. A new kind of part brings its own spec
class; nothing here needs to know it.
"""
from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm as src/model.c:164-169: w * (x / sqrt(mean(x^2) + eps)).

    one_plus: the checkpoint stores the weight around zero and the norm multiplies by 1 + w.
    """
    size: int
    eps: float
    one_plus: bool = False
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding as src/model.c:116-124, 173-181.

    pairing "half" rotates (i, i + rotary_dim/2); "interleaved" rotates (2i, 2i+1).
    rotary_dim may be smaller than the head size (the rest passes unchanged).
    """
    theta: float
    rotary_dim: int
    pairing: str = "half"
    kind: str = "rotary"
    exact_angles: bool = False  # the table's angles are made in float64 before their cosines and sines are rounded
    # Scaled frequencies (exact_angles only). linear_factor c: every frequency is divided by c. blend (factor, original,
    # fast, slow), the scaling known as YaRN: with where(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta),
    # lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), rotary_dim - 1) and
    # ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i),
    # and cosines and sines are multiplied by 0.1 ln(factor) + 1.
    linear_factor: float = 1.0
    blend: Optional[tuple] = None


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention as src/model.c:197-211, 247-259.

    window None: every earlier key; W: the last W keys, the token's own included.
    scale multiplies the scores (src/model.c:202 uses 1/sqrt(head_dim)).
    v_head_dim: the size of a value head where it is not head_dim. keep_first F (with a window): the
    sequence's first F keys stay visible behind the window, at their true positions. sink: a learned score
    per query head (slot "sink") that joins the softmax's denominator once, unscaled, with no key and no value.
    exact_weights: the softmax's weights stay float32 in the second product also where the model is bfloat16.
    conv_taps T > 0: q, k and v each pass a causal convolution of T taps per channel (no activation) right after their
    projection (slots "conv_q", "conv_k", "conv_v", [channels, taps], the last tap the token's own); the last T - 1
    projected rows are part of the sequence's state. chunk C: key j is seen from i only if i // C == j // C, positions
    counted from the sequence's first token. softcap c: score <- c * tanh(score / c), after the scale.
    norm_over "projection" (with qk_norm_eps): q and k are each normed over their whole row, all heads at once, with
    weights of that size (slots "q_norm" [heads * head_dim], "k_norm" [kv_heads * head_dim]), before the rotation.
    values "keys": there is no value projection; a value head is its key head as projected, before norm and rotation.
    head_gate: head h's output is multiplied by sigmoid(g_h . x), one number a head (slot "wg", [heads, hidden]).
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    qk_norm_eps: Optional[float]  # None: no per-head norm of q and k
    position: Optional[RotarySpec]
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    keep_first: int = 0
    sink: bool = False
    exact_weights: bool = False
    conv_taps: int = 0
    chunk: Optional[int] = None
    softcap: Optional[float] = None
    norm_over: str = "head"
    values: str = "own"
    head_gate: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """A recurrent mixer: the gated delta rule with a decay per head and key channel.

    Per head a state S [key_dim, value_dim] (float32, zero at a sequence's start):
        S <- diag(g) S;  e = b (v - S^T k);  S <- S + k e^T;  o = S^T q
    q, k (n_kv_heads x key_dim; head h uses q/k head h // (n_heads / n_kv_heads)) and v (n_heads x value_dim) each
    pass a causal convolution of conv_taps taps per channel and SiLU; q and k are then unit vectors per head
    (x / sqrt(sum x^2 + unit_eps)), q times key_dim^-1/2. b = sigmoid(.) per head. g = exp(-exp(A_h) *
    softplus(W2 (W1 x) + bias)), decay_rank the inner size of that pair of matrices. o is normed per head over
    value_dim (eps norm_eps, a weight shared by the heads) and gated by sigmoid(G2 (G1 x)), gate_rank the inner size.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    norm_eps: float
    unit_eps: float = 1e-6
    kind: str = "channel_delta"


@dataclass(frozen=True)
class HeadDeltaSpec:
    """A recurrent mixer: the gated delta rule with one decay per head.

    As DeltaRuleSpec, but g = exp(-exp(A_h) * softplus(a_h . x + bias_h)) is one number a head (slot "wa", [heads, hidden]),
    and the output gate is silu(G x) with G a full matrix [heads * value_dim, hidden].
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    kind: str = "head_delta"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """A recurrent mixer: a matrix memory per head with exponential gates kept in range by a running maximum.

    Per head q = Wq x * key_dim^-1/2, k = Wk x, v = Wv x, and two gates in the log domain,
        i = cap * tanh((wi . x + bi) / cap),    f = logsigmoid(cap * tanh((wf . x + bf) / cap)).
    State C [key, value], n [key] and a scalar m, all zero at a sequence's start (m too):
        m' = max(f + m, i);  C' = e^(f + m - m') C + e^(i - m') k v^T;  n' likewise with k alone;
        o = C'^T q / (max(|n' . q|, e^(-m')) + denom_eps).
    Each head's o is divided by its root mean square (norm_eps), the heads side by side are multiplied by a weight
    [heads * value_dim] and by sigmoid(Wg x), then projected.
    """
    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    norm_eps: float
    denom_eps: float = 1e-6
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is share * (norm(left(x); w_left) + norm(right(x); w_right)),
    each output normed over the model's width with a plain weight of its own (slots "left_out", "right_out")."""
    hidden: int
    left: object
    right: object
    norm_eps: float
    share: float = 0.5
    kind: str = "side_by_side"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are kept as one low-rank latent row per token, shared by the heads.

    Per token: q = Wq x laid out head by head as [head_dim plain | rot_dim rotated]; Wd x has rank + rot_dim rows: the
    first `rank`, normed (w * z / sqrt(mean(z^2) + norm_eps)), are the latent c, the last rot_dim one rotated key part r
    that every head shares. Head h's key is [Uk_h c | r], its value Uv_h c; the score is scale * (q . k). The cache
    holds [c | r] alone. position: a RotarySpec over (part of) the rot_dim part. sink: a learned score per head that
    joins the softmax's denominator once, unscaled, with no key and no value. shares_latents: the entry has no
    down-projection of its own and reads the cache of the schedule entry it names as its source.
    q_rank Q: the queries pass a latent of their own, q = Wuq norm(Wdq x; w) (slots "wdq" [Q, hidden], "q_norm" [Q],
    "wq" [heads * (head_dim + rot_dim), Q]). head_gate: head h's output is multiplied by sigmoid(g_h . x) (slot "wg").
    """
    hidden: int
    n_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    rank: int
    scale: float
    norm_eps: float
    position: Optional[RotarySpec]
    sink: bool = False
    shares_latents: bool = False
    q_rank: Optional[int] = None
    head_gate: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DecayAttentionSpec:
    """A recurrent mixer: linear attention with a fixed decay per head.

    q = silu(Wq x), k = silu(Wk x) (n_heads x key_dim), v = silu(Wv x) (n_heads x value_dim). Per head a float32 state
    S [key_dim, value_dim], zero at a sequence's start: S <- decay_h S + k v^T; o = S^T q. The heads' outputs, side by
    side, are normed as one row (w * o / sqrt(mean(o^2) + norm_eps)), multiplied by sigmoid(Wg x) and projected by Wo.
    """
    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay: tuple
    norm_eps: float
    kind: str = "decay_attention"


@dataclass(frozen=True)
class WkvSpec:
    """A recurrent mixer: time mixing with a decay per head, key channel and token, and a bonus for the token's own key.

    With x' the token before (zeros at a sequence's start; the last token is part of the state), each of r, k, v, g, w
    reads a blend of its own, m_s = x + (x' - x) * mu_s (slots "mu_r" ... "mu_w", [hidden]). r, k, v = W. m_.
    (n_heads x key_dim each), gate = silu(Wg m_g), decay = exp(-exp(W2 tanh(W1 m_w) + w0)) per head and key channel
    (decay_rank the inner size of that pair of matrices). Per head a float32 state S [key, value], zero at the start:
        o = (S + diag(u) k v^T)^T r;    S <- diag(decay) S + k v^T
    with the bonus u [heads, key_dim]. Each head's o is divided by its root mean square (norm_eps), the heads side by
    side are multiplied by a weight [heads * key_dim] and by the gate, then projected.
    """
    hidden: int
    n_heads: int
    key_dim: int
    decay_rank: int
    norm_eps: float
    kind: str = "wkv"


@dataclass(frozen=True)
class ExpertSpec:
    """A small feed-forward: down(act(up(x))), or, with activation "silu_gated", down(silu(gate(x)) * up(x))."""
    inter: int
    activation: str = "relu_squared"


@dataclass(frozen=True)
class RoutedMLPSpec:
    """A feed-forward of `experts` small layers of which each token uses `top`, and an optional shared one.

    Router logits z = R x in float32; score "sigmoid": s = sigmoid(z), the `top` largest chosen, weights the chosen s
    as they are; score "softmax_chosen": the softmax of the chosen logits; score "softmax_all": s = softmax(z) over
    all router outputs, the choice goes by s (plus, with correction, a learned shift per output, slot "correction", that
    the weights do not see) and the weights are the chosen s * weight_scale, not renormalized. identity I: the router has
    experts + I outputs, and the last I stand for experts without tensors whose output is their input.
    score "table": there is no router; row `token id` of an integer table (slot "table", [vocab, top]) names the token's
    experts, each with weight 1 / top.
    weight_on "input": the output is sum_e expert_e(w_e x); "output": sum_e w_e expert_e(x). shared (an ExpertSpec or
    None) runs for every token and is added.
    """
    hidden: int
    experts: int
    top: int
    expert: ExpertSpec
    shared: Optional[ExpertSpec] = None
    score: str = "sigmoid"
    weight_on: str = "input"
    correction: bool = False
    weight_scale: float = 1.0
    identity: int = 0
    vocab: int = 0  # rows of the table (score "table")
    kind: str = "routed_mlp"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) as src/model.c:274-282, 307-309."""
    hidden: int
    inter: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its two norms, its mixer, its feed-forward and how they are wired.

    arrangement "pre_norm" is src/model.c:292-310: x += mixer(norm(x)); x += ffn(norm(x)).
    """
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    arrangement: str = "pre_norm"

    @property
    def kind(self):
        return self.arrangement


@dataclass(frozen=True)
class StreamsBlockSpec:
    """One layer over a residual stream that is kept as `streams` copies X[0..s) with learned connections.

    For each branch (the mixer, then the feed-forward; ffn None: the mixer alone) with its connection
    (enter [s], mix [s, s] indexed [from, to], leave [s]):
        u = sum_s enter[s] X[s];  y = branch(norm(u));  X'[t] = sum_s mix[s, t] X[s] + branch_scale * leave[t] * y
    learned False: no connection tensors; enter = mix = leave = 1 (one stream: x += branch_scale * y).
    """
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    streams: int = 1
    branch_scale: float = 1.0
    learned: bool = True
    kind: str = "streams_pre_norm"


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """The frame "scaled_pairs": x = table[token] * scale, plus, with buckets > 0, row
    (previous token * mul_prev + token * mul_cur) mod buckets of a second table (a sequence's first token: row
    `buckets`, the last). The stream starts as `streams` copies of x and ends as their sum, normed."""
    scale: float = 1.0
    buckets: int = 0
    mul_prev: int = 0
    mul_cur: int = 0
    streams: int = 1


@dataclass(frozen=True)
class PositionEmbeddingSpec:
    """The frame "positions": x = table[token] + positions[position], a learned vector per position (slot "positions",
    [max_positions, hidden]), not scaled. keep: the frame keeps x as it leaves the embedding, for schedule entries that
    add it to the stream again (ScheduleEntry.rejoin)."""
    max_positions: int
    keep: bool = False


@dataclass(frozen=True)
class LoopInputSpec:
    """The frame "loop_input": x = table[token]; the frame keeps x as the embedding left it, and before a schedule entry
    with `inject` t the stream is made anew from itself and the embedding, x <- Win [x; x_0] + step[t] (slots "loop_in"
    [hidden, 2 hidden], x first, and "loop_step" [passes, hidden]). passes 0: no such entry, no such tensors."""
    passes: int = 0


@dataclass(frozen=True)
class ScheduleEntry:
    """One entry of the run order.

    layer: index into ModelSpec.layers (a layer may be named more than once).
    source: None if the mixer keeps keys/values or state of its own for this
    entry; else the index of an earlier entry whose cache it reads.
    rejoin: right before this entry runs, what the frame kept of the embedding is added to the stream (the frame
    must keep it). inject t: right before this entry runs, the frame makes the stream anew from the stream and the
    embedding, with its t-th step vector (LoopInputSpec).
    """
    layer: int
    source: Optional[int] = None
    rejoin: bool = False
    inject: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tied_head: bool
    max_positions: int
    stop_tokens: tuple = field(default_factory=tuple)
    frame: str = "plain"  # how tokens become the stream and the stream logits (parts/frame.py)
    frame_spec: object = None  # what that frame needs beyond the sizes above

    @property
    def kind(self):  # the frame is built from the model's spec
        return self.frame
