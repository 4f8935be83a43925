"""Descriptions of a model as data: which parts each layer is made of, with every size
and constant as a parameter, and the order in which layers run.

A *spec* is a frozen dataclass with a `kind` string.  The part registries
(`llmgen_b200.parts.registry`) map a kind to the class that runs it on the GPU, so a new
mixer, feed-forward, norm or position encoding is one spec class, one runtime class and one
`register_*` call; nothing in the engine or the cache manager changes.

The reference builds the same tree from `Ctx.config_params` and weights found by spec key
(src/module/module.zig:32-83, src/models/qwen3.zig:142-340).  Its modules append graph
nodes; ours hold device weights and launch kernels.  Tensor names are parameters of the
specs, given by the architecture's builder, so no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

# How a declared tensor is kept on the device, and how the random-weights mode draws it.
MATRIX = "matrix"      # projection or table of embeddings: compute dtype (bf16 or fp32)
VECTOR = "vector"      # norm gains and other small vectors: always fp32 on the device
INT_TABLE = "int_table"  # integer tables: int32

INIT_NORMAL = "normal"              # N(0, sigma)
INIT_ONE_PLUS_NORMAL = "one_plus"   # 1 + N(0, sigma_norm)
INIT_EYE_PLUS_NORMAL = "eye_plus"   # a square matrix: the identity + N(0, sigma_norm)


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a part reads from the model file."""
    name: str
    shape: Tuple[int, ...]
    kind: str = MATRIX
    init: str = INIT_NORMAL


# ----------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset) over the last `dim` values.

    Reference: src/module/norm.zig:49-86, src/backend/cpu/norm.zig:60-93.
    """
    dim: int
    eps: float
    weight: str
    weight_offset: float = 0.0
    kind: str = "rmsnorm"


# ----------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first `rotary_dim` values of a head, angle =
    pos / theta^(2i/rotary_dim).  `pairing` says which two values are turned together: "half" is the
    half-split (NEOX) pairing (i, i + rotary_dim/2) of the reference, "interleaved" the pairing (2i, 2i + 1); a mixer's
    kernels are told the pairing and refuse one they do not implement.

    Reference: src/module/rope.zig:60-107, src/backend/cpu/rope.zig:13-75.
    """
    rotary_dim: int
    theta: float
    max_positions: int
    pairing: str = "half"
    # Frequencies scaled by wavelength, (factor, low, high, original): with f_i = theta^(-2i/rotary_dim) and wavelength
    # l = 2 pi / f, f stays where l < original / high, becomes f / factor where l > original / low, and between the two
    # (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  None: the plain frequencies.
    scaling: Optional[Tuple[float, float, float, float]] = None
    kind: str = "rope"


# ----------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache.

    q = x Wq^T, k = x Wk^T, v = x Wv^T (no bias); optional RMSNorm over each head of q and
    of k (one gain vector shared by all heads) before the position encoding; softmax of
    q.k * scale over keys 0..pos (or the last `window` of them); output projection Wo.

    Reference: src/models/qwen3.zig:165-209, src/module/attention.zig:85-92,
    src/backend/cpu/attention.zig:64-118.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    q_norm: Optional[RMSNormSpec] = None
    k_norm: Optional[RMSNormSpec] = None
    position: Optional[RopeSpec] = None
    window: Optional[int] = None
    # Variations, all off by default.  `v_head_dim`: width of a value head where it differs from a key's.
    # `q_bias` .. `o_bias`: names of bias vectors added in the projections.  `softcap` > 0: the scaled score s
    # becomes softcap * tanh(s / softcap).  `sink`: the softmax's denominator has one more term exp(0), a key of
    # score 0 without a value, so the weights of a row sum to less than one.  `gate_proj`: the heads side by side
    # are multiplied by sigmoid(x Wg^T) before the output projection.
    v_head_dim: Optional[int] = None
    q_bias: Optional[str] = None
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    o_bias: Optional[str] = None
    softcap: float = 0.0
    sink: bool = False
    gate_proj: Optional[str] = None
    # `unit_norm_eps`: after the rotation, every head of q and k is divided by its root mean square,
    # x / sqrt(mean(x^2) + unit_norm_eps), without gains (in place of `q_norm` / `k_norm`, which come before the rotation).
    # `chunk`: a query sees the keys at or before it that lie in its own block of `chunk` positions,
    # floor(j / chunk) = floor(i / chunk), blocks counted from the sequence's first position.
    unit_norm_eps: Optional[float] = None
    chunk: Optional[int] = None
    # `conv`: a short causal convolution over time on every channel of q, k and v, straight after the projections (one
    # spec over the channels of q, k and v side by side; `conv_weights` names the three tensors of taps, stacked when the
    # model is loaded); the sequence's last taps - 1 projected rows are state.  `row_norms`: `q_norm` / `k_norm` run over the
    # whole projection of a token (all heads at once, gains of that size) instead of over each head.  `rotate_values`: the
    # value of position j is turned by j over all of its width in half-split pairs (frequencies theta^(-2m / value width),
    # theta the position encoding's) before it is cached, and each head's output at position i is turned back by -i.
    # `sink_scores`: with `sink`, the name of a tensor [heads] of learned sink scores (the term is exp(score_h)).
    # `gate_per_head`: `gate_proj` is [heads, hidden], one number per head.
    conv: Optional["ShortConvSpec"] = None
    conv_weights: Tuple[str, ...] = ()
    row_norms: bool = False
    rotate_values: bool = False
    sink_scores: Optional[str] = None
    gate_per_head: bool = False
    kind: str = "attention"

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass(frozen=True)
class LinearAttentionSpec:
    """Linear attention with a decay per head and a state carried from token to token.

    q = act(x Wq^T), k = act(x Wk^T) [heads, key_dim], v = act(x Wv^T) [heads, value_dim]; per head
    S_t = decay_h S_(t-1) + k_t (x) v_t (float32, zero when the request starts), o_t = S_t^T q_t, no other scale.
    The heads side by side pass an RMSNorm (`out_norm`, optional), are multiplied by sigmoid(x Wg^T) (`gate_proj`,
    optional) and projected by Wo.  The state [heads, key_dim, value_dim] lives in the cache manager's state slots.
    """
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]             # one factor per head
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    gate_proj: Optional[str] = None
    out_norm: Optional[RMSNormSpec] = None
    activation: str = "silu"             # on q, k and v: "silu" or "none"
    kind: str = "linear_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are expanded from a cached latent vector per token.

    Queries through a latent of their own: cq = norm(x Wdq^T), q = cq Wuq^T, per head [nope_dim | rope_dim].
    x Wdkv^T has kv_rank + rope_dim values: the first kv_rank, normed, are the latent c; the last rope_dim are one
    rotated key part shared by all heads.  Head h: key [Wuk_h c | rotated part], value Wuv_h c (value_dim);
    score = (q . key) * scale.  The heads side by side are multiplied by sigmoid(x Wg^T) (`gate_proj`, optional) and
    projected by Wo.  Only [c | rotated part] is cached (one shared entry of kv_rank + rope_dim values per token).
    """
    hidden_size: int
    num_heads: int
    nope_dim: int
    rope_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    dq_proj: str
    uq_proj: str
    dkv_proj: str
    uk_proj: str
    uv_proj: str
    o_proj: str
    q_norm: RMSNormSpec
    kv_norm: RMSNormSpec
    position: Optional[RopeSpec] = None
    gate_proj: Optional[str] = None
    # fold Wuk into the query's up-projection when the model is loaded (one product straight into the latent space
    # instead of a product and a per-head product); False keeps the two matrices apart
    absorb_at_load: bool = True
    kind: str = "latent_attention"


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time on each channel by itself: out_t = sum_j taps[:, j] in_(t - (K-1) + j) + bias,
    taps [channels, K] with the last column on the current token, zeros before the first token of a sequence.  The last
    K - 1 inputs of a sequence are part of its mixer's state."""
    channels: int
    taps: int
    weight: str
    bias: Optional[str] = None


@dataclass(frozen=True)
class RGLRUSpec:
    """A recurrent block around a real-gated linear recurrent unit.

    Two branches of `width` channels off the mixer's input: y = gelu_tanh(x Wy^T + by) and u = conv(x Wx^T + bx).
    The channels are cut into `blocks` equal parts; in part b, r = sigmoid(Ra_b u_b + ba_b) and i = sigmoid(Ri_b u_b + bi_b)
    with square matrices per part.  a = exp(-decay_scale * r * softplus(lam)), S_t = a S_(t-1) + sqrt(1 - a^2) (i u),
    S float32 and zero before the first token; output (S * y) Wo^T.  State per request: S and the convolution's last
    taps - 1 inputs."""
    hidden_size: int
    width: int
    blocks: int
    conv: ShortConvSpec
    y_proj: str
    x_proj: str
    o_proj: str
    a_gate: str                          # [blocks, n, n], n = width / blocks
    i_gate: str
    lam: str                             # [width]
    y_bias: Optional[str] = None
    x_bias: Optional[str] = None
    a_gate_bias: Optional[str] = None    # [blocks, n]
    i_gate_bias: Optional[str] = None
    decay_scale: float = 8.0
    kind: str = "rglru"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule with a decay per head and key channel, state carried from token to token.

    q, k [kv_heads, key_dim] and v [heads, value_dim] are projections that pass a short convolution (one spec over
    the channels of q, k and v side by side) and silu; q and k are then unit vectors per head, x / sqrt(sum x^2 + unit_eps),
    and q is multiplied by key_dim^(-1/2).  Head h reads q/k head h // (heads / kv_heads).  beta = sigmoid(x Wb^T) per head.
    g = exp(-exp(A_log_h) * softplus(x Wa1^T Wa2^T + dt_bias)) [heads, key_dim].  Per head, S [key_dim, value_dim] float32,
    zero before the first token:  S <- diag(g) S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q.
    Each head's o passes an RMSNorm over value_dim (`out_norm`, one gain vector for all heads), is multiplied by
    sigmoid(x Wg1^T Wg2^T) and projected by Wo.  State per request: S and the convolution's last taps - 1 inputs."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv: ShortConvSpec                  # channels = 2 kv_heads key_dim + heads value_dim
    conv_weights: Tuple[str, ...]        # the taps of q, k and v, stacked into `conv` when the model is loaded
    q_proj: str
    k_proj: str
    v_proj: str
    beta_proj: str
    decay_down: str                      # Wa1 [rank, hidden]
    decay_up: str                        # Wa2 [heads key_dim, rank]
    decay_bias: str                      # dt_bias [heads key_dim]
    decay_log: str                       # A_log [heads]
    gate_down: str                       # Wg1
    gate_up: str                         # Wg2 [heads value_dim, rank]
    o_proj: str
    out_norm: RMSNormSpec
    decay_rank: int = 0
    gate_rank: int = 0
    unit_eps: float = 1e-6
    kind: str = "gated_delta"


@dataclass(frozen=True)
class ChannelDecayAttentionSpec:
    """Linear attention whose state forgets by a decay per head and key channel that the token itself decides.

    q = x Wq^T * key_dim^(-1/2), k = x Wk^T [heads, key_dim], v = x Wv^T [heads, value_dim]; the decay
    a = sigmoid(z)^(1 / tau), z = (x Wa1^T) Wa2^T + bias, [heads, key_dim].  Per head, S [key_dim, value_dim] float32, zero
    before the first token:  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t.  Each head's o passes an RMSNorm over
    value_dim (`out_norm`, one gain vector for all heads), the heads side by side are multiplied by silu(x Wg^T) and projected
    by Wo.  State per request: S."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    tau: float
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    decay_down: str                      # Wa1 [rank, hidden]
    decay_up: str                        # Wa2 [heads key_dim, rank]
    decay_bias: str                      # [heads key_dim]
    out_norm: RMSNormSpec
    decay_rank: int = 16
    kind: str = "channel_decay_attention"


@dataclass(frozen=True)
class TokenShiftDecaySpec:
    """Time mixing over blends of each token with the one before it, with a decay per head and key channel and a bonus
    for the token's own key.

    With x' the row of the token before (zeros before the first), each of r, k, v, g, w reads its own blend
    m_s = x + (x' - x) mu_s.  r, k, v = W m [heads, head_dim]; gate = silu(Wg m_g); the decay
    w = exp(-exp(Ww2 tanh(Ww1 m_w) + w0)) [heads, head_dim].  Per head, S [head_dim, head_dim] float32, zero before the
    first token:  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,  S_t = diag(w_t) S_(t-1) + k_t v_t^T.  Each head's o is divided by
    its root mean square (eps inside the root); the heads side by side are multiplied by `out_gain`, by the gate, and
    projected by Wo.  State per request: S and the last row of x."""
    hidden_size: int
    num_heads: int
    head_dim: int
    eps: float
    mix: Tuple[str, str, str, str, str]  # mu of r, k, v, g, w: [hidden] each
    r_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    decay_down: str                      # Ww1 [rank, hidden]
    decay_up: str                        # Ww2 [heads head_dim, rank]
    decay_bias: str                      # w0 [heads head_dim]
    bonus: str                           # u [heads, head_dim]
    out_gain: str                        # [heads head_dim]
    decay_rank: int = 16
    kind: str = "token_shift_decay"


@dataclass(frozen=True)
class MinGRUSpec:
    """A gated recurrence per channel whose gates read the current token only.

    z = sigmoid(x Wz^T + bz), u = x Wx^T + bx, both `width` wide; the candidate is u + 1/2 where u >= 0 and sigmoid(u) below;
    S_t = (1 - z_t) S_(t-1) + z_t candidate_t, float32, zero before the first token; output (S_t * silu(x Wg^T)) Wo^T.
    State per request: S."""
    hidden_size: int
    width: int
    z_proj: str
    x_proj: str
    gate_proj: str
    o_proj: str
    z_bias: Optional[str] = None
    x_bias: Optional[str] = None
    kind: str = "min_gru"


@dataclass(frozen=True)
class MLSTMSpec:
    """A matrix memory per head with exponential gates held in range by a running maximum.

    q = x Wq^T key_dim^(-1/2), k = x Wk^T [heads, key_dim], v = x Wv^T [heads, value_dim]; per head the log gates
    i = cap tanh((x Wi^T + bi) / cap) and f = logsigmoid(cap tanh((x Wf^T + bf) / cap)).  With m_0 = 0, S_0 = 0, n_0 = 0:
    m_t = max(f + m_(t-1), i);  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t the same with k alone;
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps).  Each head's o is divided by its root mean square (eps), the heads
    side by side are multiplied by `out_gain` [heads value_dim] and sigmoid(x Wg^T), and projected by Wo.  State per request:
    S, n and m, float32."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    i_proj: str
    f_proj: str
    gate_proj: str
    o_proj: str
    out_gain: str
    i_bias: Optional[str] = None
    f_bias: Optional[str] = None
    den_eps: float = 1e-6
    kind: str = "mlstm"


@dataclass(frozen=True)
class GeneralDeltaSpec:
    """The delta rule with a decay per head and key channel and a removal rate of its own.

    r, k, v = x W^T [heads, head_dim].  w = exp(-decay_scale sigmoid(tanh(x Ww1^T) Ww2^T + w0)) and a = sigmoid(x Wa^T + a0), both
    [heads, head_dim]; u = k / sqrt(sum k^2 + unit_eps) per head.  Per head, S [head_dim, head_dim] float32, zero before the first
    token:  S_t = diag(w) S_(t-1) - (a u)(u^T S_(t-1)) + k v^T;  o = S_t^T r.  Each head's o is divided by its root mean square (eps),
    the heads side by side are multiplied by `out_gain` [heads head_dim] and sigmoid(x Wg^T), and projected by Wo.  State per
    request: S."""
    hidden_size: int
    num_heads: int
    head_dim: int
    eps: float
    r_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    o_proj: str
    removal_proj: str                    # Wa [heads head_dim, hidden]
    removal_bias: str                    # a0 [heads head_dim]
    decay_down: str                      # Ww1 [rank, hidden]
    decay_up: str                        # Ww2 [heads head_dim, rank]
    decay_bias: str                      # w0 [heads head_dim]
    out_gain: str
    decay_rank: int = 16
    decay_scale: float = 0.6065306597126334      # exp(-1/2)
    unit_eps: float = 1e-6
    kind: str = "general_delta"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side that read the same input: the result is sum_i scales[i] * branches[i](x).  At most
    one branch keeps paged keys and values; the states of the branches that keep one lie side by side in one row."""
    branches: Tuple[object, ...]
    scales: Tuple[float, ...]
    kind: str = "parallel"


# ---------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class DenseMLPSpec:
    """Feed-forward without a gate: down( act(x Wup^T) ), act = relu(.)^2 ("relu2") or the tanh form of gelu ("gelu_tanh")."""
    hidden_size: int
    intermediate_size: int
    up_proj: str
    down_proj: str
    activation: str = "relu2"
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class ClampedExpertSpec:
    """One small gated feed-forward with clamped branches: g = min(x Wgate^T, limit), u = clamp(x Wup^T, -limit, limit),
    y = g sigmoid(alpha g) (u + 1), output y Wdown^T; no biases."""
    intermediate_size: int
    limit: float
    gate_proj: str
    up_proj: str
    down_proj: str
    alpha: float = 1.702


@dataclass(frozen=True)
class GatedExpertSpec:
    """One small gated feed-forward: (act(x Wgate^T) * (x Wup^T)) Wdown^T, act = silu; no biases."""
    intermediate_size: int
    gate_proj: str
    up_proj: str
    down_proj: str
    activation: str = "silu"


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of experts: router scores s = sigmoid(x Wr^T + b) (or softmax) in float32, the `top_k` largest choose
    experts, their scores are the weights (renormalised over the chosen ones if `renormalize`); with scoring
    "softmax_top" the logits themselves choose and the weights are the softmax over the chosen logits alone.  The weight
    multiplies the expert's input (`weight_on_input`) or its output.  An optional shared expert runs for every token and
    is added.  Experts are `ClampedExpertSpec` or `GatedExpertSpec`, all routed ones of one kind and size."""
    hidden_size: int
    router: str
    experts: Tuple[object, ...]
    top_k: int
    shared: Optional[object] = None
    scoring: str = "sigmoid"
    renormalize: bool = False
    weight_on_input: bool = True
    router_bias: Optional[str] = None
    kind: str = "routed_mlp"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down( act(x Wg^T) * (x Wu^T) ).

    Reference: src/models/qwen3.zig:142-163 (SwiGLU: act = x / (1 + exp(-x)),
    src/backend/cpu/activation.zig:13-17).
    """
    hidden_size: int
    intermediate_size: int
    gate_proj: str
    up_proj: str
    down_proj: str
    activation: str = "silu"             # "silu" or "gelu_tanh"
    kind: str = "gated_mlp"


# ----------------------------------------------------------------------------- blocks
@dataclass(frozen=True)
class PreNormBlockSpec:
    """x1 = x + mixer(norm(x)); x2 = x1 + ffn(norm(x1)).  `ffn` (and `ffn_norm`) may be None: a layer without a
    feed-forward stops after the first sum.

    Reference: src/models/qwen3.zig:211-237.
    """
    mixer_norm: object
    mixer: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    kind: str = "prenorm"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """x1 = x + norm(mixer(x)); x2 = x1 + norm(ffn(x1)): the norms sit on the sublayers' outputs and the sublayers
    read the residual stream itself.  `ffn` (and `ffn_norm`) may be None: a layer without a feed-forward."""
    mixer_norm: object
    mixer: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    kind: str = "postnorm"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x1 = x + norm_b(mixer(norm_a(x))); x2 = x1 + norm_d(ffn(norm_c(x1))): a norm on each sublayer's input and another on
    its output.  `ffn` (with its two norms) may be None: a layer without a feed-forward."""
    mixer_norm: object
    mixer: object
    mixer_out_norm: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    ffn_out_norm: Optional[object] = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class StreamCoefficients:
    """How one sublayer of a `MultiStreamBlockSpec` reads and writes the streams: tensors `read` [streams], `write` [streams] and
    `mix` [streams, streams] (indexed [from, to])."""
    read: str
    write: str
    mix: str


@dataclass(frozen=True)
class MultiStreamBlockSpec:
    """A pre-norm layer over `streams` residual streams x_1 .. x_S per token (hyper-connections), all equal to the embedding's
    output before the first layer and added up after the last.  Sublayer q (the mixer, then the feed-forward) with its
    coefficients:  u = sum_s read[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s mix[s, t] x_s + residual_mult write[t] y for all t
    at once, from the old streams.  Without coefficients (`mixer_streams` / `ffn_streams` None; `streams` is then 1) a sublayer
    is the plain x <- x + residual_mult sublayer(norm(x)).  `ffn` (with its norm and coefficients) may be None."""
    mixer_norm: object
    mixer: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    streams: int = 1
    residual_mult: float = 1.0
    mixer_streams: Optional[StreamCoefficients] = None
    ffn_streams: Optional[StreamCoefficients] = None
    kind: str = "multi_stream"


@dataclass(frozen=True)
class ReentrySpec:
    """What happens to the residual stream before a run item: x <- [x | x0] W^T + table[row], with x0 the embedding's
    output of the same token, W [hidden, 2 hidden] (the stream's columns first) and `table` [rows, hidden]."""
    proj: str
    table: str
    row: int
    rows: int
    kind: str = "reentry"


@dataclass(frozen=True)
class RunItem:
    """One entry of the run list: run `layer`, with cache number `cache`.

    A layer may be named by several items (each with a cache of its own or a shared one),
    and an item with `writes_cache=False` reads the cache that another item filled in the
    same step.  `cache` is None for a layer that keeps nothing between steps.  `before`: a `ReentrySpec`
    applied to the residual stream before the layer runs.
    """
    layer: int
    cache: Optional[int]
    writes_cache: bool = True
    before: Optional[ReentrySpec] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, run list, final norm, output projection."""
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str                       # name of the [vocab, hidden] table
    layers: Tuple[object, ...]           # block specs
    run_order: Tuple[RunItem, ...]
    final_norm: object
    lm_head: str                         # same name as `embedding` when tied
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    init_sigma: float = 0.02             # defaults of the random-weights mode
    init_sigma_norm: float = 0.1
    embedding_scale: float = 1.0         # rows of the table are multiplied by this as they enter the residual
    logit_cap: float = 0.0               # > 0: logits = cap * tanh(logits / cap)
    logit_scale: float = 1.0             # logits are multiplied by this (before the cap)
    embedding_norm: Optional[object] = None   # a norm spec: the embedding's rows pass it before they become the residual
    # > 0: the layers keep this many residual streams per token (`MultiStreamBlockSpec`): the model hands them a float32
    # [tokens, streams, hidden] array, every stream the embedding's output, and adds the streams up before the final norm
    residual_streams: int = 0
    # Tensors that a model folder of this architecture may carry although the model reads none of them
    # (shell patterns), and (name, declared name) pairs of such tensors that must then hold the same values.
    ignorable_tensors: Tuple[str, ...] = ()
    same_as: Tuple[Tuple[str, str], ...] = ()

    @property
    def tied(self) -> bool:
        return self.lm_head == self.embedding


def default_run_order(num_layers: int) -> Tuple[RunItem, ...]:
    return tuple(RunItem(layer=i, cache=i) for i in range(num_layers))
