"""Descriptions of a model as data: which parts each layer is made of, with every size and
constant as a parameter, and the order in which layers run.

A description is built from a typed configuration by the architecture's `describe` function; no
part class is touched until the model is built. Each spec names its `kind`; the part registry
(parts/registry.py) maps (category, kind) to the class that implements it, so a new mixer,
feed-forward, norm or position encoding is a new spec class plus one registered part class, and a
model may use different kinds in different layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Optional, Tuple


@dataclass(frozen=True)
class TensorNeed:
    """One checkpoint tensor a part reads.
    precision: "compute" = a matrix that feeds matrix products, kept in the engine's dtype
               (bfloat16, or float32 on the 32-bit path);
               "float32" = always widened to float32 (norm weights and other vectors);
               "stored"  = kept as the file stores it (32-bit stays 32-bit, integer tables int32).
    init: what the random-weights mode draws for it: "normal" = N(0, std); "around_one" = N(1, std)
          (weights that multiply, such as a norm's); "zeros" (biases and other additive terms)."""
    name: str
    shape: Tuple[int, ...]
    precision: str = "compute"
    init: str = "normal"


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": x / sqrt(mean(x^2) + eps) * weight. kind "rmsnorm_unit_offset": the same with the weight stored around
    zero and applied as (1 + weight). kind "layernorm": (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight, no bias."""
    kind: str
    dim: int
    eps: float
    weight: str  # checkpoint tensor name


@dataclass(frozen=True)
class PositionSpec:
    """kind "rope": rotary, half-split layout over `head_dim` numbers (a mixer that rotates only the first numbers of a head
    names that count here); `scaling` as in the configuration: with l = 2 pi / f and original_max_positions > 0, f stays where
    l < original / high_freq_factor, becomes f / scaling_factor where l > original / low_freq_factor, and between the two is
    (1 - s) f / scaling_factor + s f with s = (original / l - low) / (high - low). float64_frequencies: the frequencies enter
    the angles as float64 numbers instead of being rounded to float32 first (the reference's tables round them). kind "none"."""
    kind: str
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling_factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_positions: int = 0  # 0: no rescaling of frequencies
    float64_frequencies: bool = False


@dataclass(frozen=True)
class ScaledRotarySpec:
    """kind "rope_ramp": rotary, half-split layout over the first `dims` numbers of the vector it is given.
    Pair i turns by position * f_i, f_i = base^(-2i/dims). With factor > 0 the frequencies are stretched
    along a ramp: turn(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turn(fast)), 0),
    hi = min(ceil(turn(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are both multiplied by
    0.1 ln(factor) + 1. factor 0: plain frequencies, no multiplier."""
    kind: str
    dims: int
    base: float
    max_positions: int
    factor: float = 0.0
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are maps of one cached latent per token (parts/latent_attention.py).
    heads H; per head `dim` unrotated and `rot_dim` rotated query/key numbers and `vdim` value numbers;
    `kv_rank` the latent of keys and values, `q_rank` the latent of queries. `scale` multiplies the scores as given."""
    kind: str
    hidden: int
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    eps: float
    position: object  # a position spec with rotation tables over `dims` <= rot_dim numbers
    dq_weight: str
    dq_norm: str
    uq_weight: str
    dkv_weight: str
    dkv_norm: str
    uk_weight: str
    uv_weight: str
    gate_weight: str
    o_weight: str
    window: int = 0


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention. window = 0 keeps every key; W > 0 reads the last W."""
    kind: str
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: PositionSpec
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    window: int = 0
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Causal grouped-query attention with keys of `head_dim` and values of `value_dim` numbers a head (kind "gated_attention",
    parts/gated_attention.py). Options, each off when its field is None / 0 / False:
    q_norm, k_norm: RMS norm of every query / key head over head_dim with one weight [head_dim] for all heads, before the rotation;
    position: a position spec with rotation tables over the first `dims` <= head_dim numbers of a head;
    chunk: position i sees j <= i only if floor(i / chunk) == floor(j / chunk) (chunk borders are absolute positions);
    window: the last `window` keys; sink: a number per head whose exponential is one more term of the softmax's denominator;
    value_mix: "first" = this layer's values are kept for the step's tokens, "mix" = v <- (1 - m) v + m v_first with the scalar
    tensor `value_mix_weight` and the values of the step's "first" layer (the mixed values are cached);
    gate_weight: the heads' outputs are multiplied by sigmoid(Wg h) before the output projection.
    norm_scope "projection": q_norm [num_heads * head_dim] and k_norm [num_kv_heads * head_dim] are weights of ONE RMS norm over all
    query heads' numbers together and one over all key heads', in place of a norm a head.
    own_kv False: the layer has no key and value projections (no k_weight, v_weight, k_norm): its run reads the cache of the run that
    LayerRun.cache_from names, keys as that layer normalised and rotated them. cache_window: how many of the last keys the cache
    must keep when that is more than this layer's own window asks for, because borrowers look further back (None: `window`; 0: all)."""
    kind: str
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    position: object
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    sink: Optional[str] = None
    gate_weight: Optional[str] = None
    value_mix: Optional[str] = None        # None | "first" | "mix"
    value_mix_weight: Optional[str] = None
    chunk: int = 0
    window: int = 0
    gate_per_head: bool = False            # the gate is one number a head (gate_weight [heads, hidden]) instead of one a result number
    norm_scope: str = "head"               # "head" | "projection"
    own_kv: bool = True
    cache_window: Optional[int] = None


@dataclass(frozen=True)
class SelectiveScanSpec:
    """A recurrent mixer with input-dependent decay (kind "selective_scan", parts/selective_scan.py): [x | z] = W_in h;
    x <- silu(causal convolution over `taps` inputs a channel, with bias); [dt_low: dt_rank | B: state | C: state] = W_x x;
    dt = softplus(W_dt dt_low + dt_bias); S <- exp(dt A) S + dt x B, A = -exp(a_log); y = S C + skip x; out = W_o (y silu(z)).
    The state (S [inner, state] and the convolution's last taps - 1 inputs) is float32 and kept per request."""
    kind: str
    hidden: int
    inner: int
    state: int
    taps: int
    dt_rank: int
    in_weight: str
    conv_weight: str
    conv_bias: str
    x_weight: str
    dt_weight: str
    dt_bias: str
    a_log: str
    skip: str
    o_weight: str


@dataclass(frozen=True)
class DecayedLinearAttentionSpec:
    """A recurrent mixer with a matrix of state per head and a decay per key channel (kind "decayed_linear_attention",
    parts/linear_state.py): q = Wq h * dim^(-1/2), k = Wk h (heads x dim), v = Wv h (heads x vdim);
    a = sigmoid(W_a2 (W_a1 h) + a_bias)^(1 / tau) per head and key channel; S <- diag(a) S + k v^T; o = S^T q; every head's o is
    divided by its root mean square (eps) and multiplied by norm_weight [vdim]; out = Wo (o * silu(Wg h))."""
    kind: str
    hidden: int
    heads: int
    dim: int
    vdim: int
    rank: int
    tau: float
    eps: float
    q_weight: str
    k_weight: str
    v_weight: str
    g_weight: str
    o_weight: str
    norm_weight: str
    a1_weight: str
    a2_weight: str
    a2_bias: str


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with one fixed decay per head and neither softmax nor denominator (kind "retention", parts/linear_state.py):
    q = Wq h, k = Wk h (heads x dim), v = Wv h (heads x vdim); q and k rotated by `position` (any position spec with rotation tables
    over the first numbers of a head); k times k_scale after the rotation; S <- decay_h S + k v^T; o = S^T q; every head's o is divided by
    its root mean square (eps, no weight); out = Wo (o * silu(Wg h))."""
    kind: str
    hidden: int
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    k_scale: float
    eps: float
    position: object
    q_weight: str
    k_weight: str
    v_weight: str
    g_weight: str
    o_weight: str


@dataclass(frozen=True)
class TokenShiftMixSpec:
    """A recurrent mixer whose projections read blends of a token's input with the previous token's (kind "token_shift_mix",
    parts/linear_state.py): x_s = h + (h_prev - h) * mu_s for s in r, k, v, g, w; r, k, v = W x (heads x dim); gate =
    silu(Wg x_g); decay = exp(-exp(W_w2 tanh(W_w1 x_w) + w0)) per head and key channel; o = (S + diag(bonus) k v^T)^T r, then
    S <- diag(decay) S + k v^T; every head's o is divided by its root mean square (eps); out = Wo (o * norm_weight * gate)."""
    kind: str
    hidden: int
    heads: int
    dim: int
    rank: int
    eps: float
    mu: Tuple[str, ...]  # the blends' weights, in the order r, k, v, g, w
    r_weight: str
    k_weight: str
    v_weight: str
    g_weight: str
    o_weight: str
    w1_weight: str
    w2_weight: str
    w0: str
    bonus: str
    norm_weight: str


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule behind short convolutions (kind "gated_delta", parts/linear_state.py): q, k = W h (kv_heads x dim),
    v = W h (heads x vdim), each through a causal convolution of `taps` inputs a channel (no bias) and silu; q and k made unit
    vectors per head (x / sqrt(sum x^2 + unit_eps)), q times dim^(-1/2); beta = sigmoid(Wb h), g = exp(-exp(a_log) *
    softplus(Wa h + dt_bias)) per head; S <- g S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q; every head's o is divided by
    its root mean square (eps) and multiplied by norm_weight [vdim]; out = Wo (o * silu(Wg h))."""
    kind: str
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    eps: float
    q_weight: str
    k_weight: str
    v_weight: str
    q_conv: str
    k_conv: str
    v_conv: str
    b_weight: str
    a_weight: str
    a_log: str
    dt_bias: str
    g_weight: str
    norm_weight: str
    o_weight: str
    unit_eps: float = 1e-6


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers side by side that read the same input (kind "mixer_pair", parts/mixer_pair.py). combine "weighted":
    left_scale * left + right_scale * right. combine "normed_mean": (rms(left) * left_norm + rms(right) * right_norm) / 2, the
    root mean square over the model width (eps inside the root), the weights [hidden] as stored."""
    kind: str
    hidden: int
    left: object
    right: object
    combine: str = "weighted"
    left_scale: float = 1.0
    right_scale: float = 1.0
    left_norm: Optional[str] = None
    right_norm: Optional[str] = None
    eps: float = 0.0


@dataclass(frozen=True)
class GatedMLPSpec:
    """down( act(gate(x)) * up(x) ), dense, no bias. activation "silu" or "gelu_tanh"; "clamped_swish": g = min(gate(x), limit),
    u = clamp(up(x), -limit, limit), down(g * sigmoid(slope * g) * (u + 1))."""
    kind: str
    hidden: int
    intermediate: int
    gate_weight: str
    up_weight: str
    down_weight: str
    activation: str = "silu"
    limit: float = 0.0
    slope: float = 1.0


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of experts: logits = router x + router_bias in float32; each token uses the `top` experts with the largest
    logits, weighted by the softmax over the chosen logits; an expert is down_e(act(up_e(x))) without biases.
    up_weights / down_weights: one checkpoint name per expert. activation "gelu" (the exact, erf form)."""
    kind: str
    hidden: int
    intermediate: int
    experts: int
    top: int
    router_weight: str
    router_bias: Optional[str]
    up_weights: Tuple[str, ...]
    down_weights: Tuple[str, ...]
    activation: str = "gelu"


@dataclass(frozen=True)
class GroupRoutedMLPSpec:
    """Mixture of gated experts with scores over all experts (kind "group_routed_mlp"): s = softmax(router x) in float32, or
    (score "sigmoid") the sigmoid of every logit; choice scores = s + correction (optional tensor [experts]); the experts form
    `groups` equal groups of neighbours, a group's score is its largest choice score (group_top 1) or the sum of its two largest
    (group_top 2), and only experts of the best `keep_groups` groups can be chosen; the `top` largest choice scores win; their
    weights are s (without the correction) divided by (their sum + norm_eps), or s as it is (normalize False), then times
    weight_scale; an expert is down_e(act(gate_e x) * up_e x) without biases (activation "silu", or "clamped_swish" with `limit`
    and `slope` as in GatedMLPSpec); `shared` (a GatedMLPSpec or None) runs for every token and is added, times
    sigmoid(shared_gate . x) (a tensor [1, hidden]) if shared_gate names one. identity: the router has `experts + identity`
    outputs, and the last `identity` of them are experts without tensors whose result is the input x itself (scores, correction,
    groups and the choice run over all experts + identity outputs)."""
    kind: str
    hidden: int
    intermediate: int
    experts: int
    top: int
    router_weight: str
    correction: Optional[str]
    gate_weights: Tuple[str, ...]
    up_weights: Tuple[str, ...]
    down_weights: Tuple[str, ...]
    groups: int = 1
    keep_groups: int = 1
    norm_eps: float = 1e-20
    activation: str = "silu"
    shared: object = None
    score: str = "softmax"
    group_top: int = 1
    normalize: bool = True
    weight_scale: float = 1.0
    identity: int = 0
    shared_gate: Optional[str] = None
    limit: float = 0.0
    slope: float = 1.0


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, added after the layer: e = table[token, col0 : col0 + dim];
    y = proj(gelu_tanh(gate(x)) * e) for the stream x; x += y / rms(y) * norm (eps inside the root)."""
    kind: str
    hidden: int
    dim: int
    vocab_size: int
    table: str       # [vocab, table_width], shared by all layers
    table_width: int
    col0: int
    gate_weight: str  # [dim, hidden]
    proj_weight: str  # [hidden, dim]
    norm_weight: str  # [hidden]
    eps: float


@dataclass(frozen=True)
class BlockSpec:
    """kind "pre_norm": h += mixer(norm1(h)); h += feed_forward(norm2(h)).
    kind "parallel": h += mixer(norm1(h)) + feed_forward(norm2(h)), both of the same h (feed_forward and norm2 may be
    None: then the mixer alone; norm2 None with a feed_forward: ONE norm, and both sub-layers read norm1(h)); then, if
    `token_input` is given, h += token_input(h, tokens).
    kind "post_norm": the norms sit on the sub-layers' outputs and the sub-layers read h itself:
    h += scale1 * norm1(mixer(h)); h += scale2 * norm2(feed_forward(h)) (feed_forward and norm2 may be None); scale1 / scale2 name
    optional per-column layer-scale tensors [hidden].
    kind "sandwich": a norm before and one after each sub-layer: h += residual_mult * norm1_out(mixer(norm1(h)));
    h += residual_mult * norm2_out(feed_forward(norm2(h))) (feed_forward, norm2 and norm2_out may be None).
    mixer / feed_forward / token_input are any registered spec objects with a `kind`."""
    kind: str
    norm1: object
    mixer: object
    norm2: object
    feed_forward: object
    token_input: object = None
    scale1: Optional[str] = None
    scale2: Optional[str] = None
    norm1_out: object = None
    norm2_out: object = None
    residual_mult: float = 1.0


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run `layer`; if `cache_from` names another layer, this
    run reads that layer's cache and writes none of its own. add_embedding: the embedding's output
    (the stream as it was before the first run) is added to the stream right before this run."""
    layer: int
    cache_from: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class EmbeddingSpec:
    """kind "lookup": residual stream row = table row of the token id, widened to float32, times `scale`.
    kind "lookup_normed": the same, then `norm` (any norm spec over `dim`) applied to the row: the stream starts normalised."""
    weight: str
    vocab_size: int
    dim: int
    kind: str = "lookup"
    scale: float = 1.0
    norm: object = None


@dataclass(frozen=True)
class HeadSpec:
    """kind "linear": logits = x . W^T in float32, no bias, for the wanted rows only; with softcap c > 0 then
    logits <- c * tanh(logits / c)."""
    weight: str  # the embedding's name when input and output embeddings are tied
    vocab_size: int
    dim: int
    kind: str = "linear"
    softcap: float = 0.0


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: object  # any registered "embedding" spec with `kind`, `weight`, `vocab_size`, `dim`
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerRun, ...]
    final_norm: object
    head: object       # any registered "head" spec with `kind`, `weight`, `vocab_size`, `dim`
    max_positions: int
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)
    # names that may be present in the checkpoint without being read, each with the needed tensor
    # it must agree with in shape (a tied lm_head saved beside the embedding)
    duplicates: Dict[str, str] = field(default_factory=dict)
    # shell-style patterns of names that a checkpoint may carry and nobody reads (buffers that some
    # exporters save, such as "*.rotary_emb.inv_freq"); the reference maps whatever a file holds and
    # reads what it needs (src/weights.cpp:269-301), so it ignores them too
    ignore: Tuple[str, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.head.vocab_size

    @property
    def hidden_size(self) -> int:
        return self.embedding.dim
