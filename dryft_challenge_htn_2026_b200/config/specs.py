"""Specifications of parts and of a whole model.

A specification is plain data: the sizes and constants a part needs, nothing about the model it
ends up in. An architecture's config class turns its config.json into a ``ModelSpec``; the parts
registry (``parts.registry``) turns each specification into the part that runs it. A new kind of
mixer, feed-forward, norm or position encoding is a new specification class plus a part class
registered for it; nothing in this file has to change.
"""
from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = w * x * rsqrt(mean(x^2) + eps) over the last ``dim`` elements. ``tensor``: the weight's name under the
    part's prefix (empty: the prefix itself names it)."""
    dim: int
    eps: float
    tensor: str = "weight"


@dataclass(frozen=True)
class ScalarRMSNormSpec:
    """y = g * x * rsqrt(mean(x^2) + eps) with one learned number g for all ``dim`` coordinates."""
    dim: int
    eps: float


@dataclass(frozen=True)
class OnePlusRMSNormSpec:
    """y = (1 + w) * x * rsqrt(mean(x^2) + eps): an RMS norm whose stored weight sits around zero."""
    dim: int
    eps: float


@dataclass(frozen=True)
class UnitRMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) over the last ``dim`` elements: an RMS norm without a weight."""
    dim: int
    eps: float


@dataclass(frozen=True)
class GroupRMSNormSpec:
    """RMS norm in groups: the ``dim`` coordinates are split into ``groups`` equal consecutive parts, each part is
    divided by its own sqrt(mean(part^2) + eps), and the whole is multiplied by a weight of size ``dim``. ``tensor``:
    the weight's name under the part's prefix (empty: the prefix itself names it)."""
    dim: int
    eps: float
    groups: int = 1
    tensor: str = ""


@dataclass(frozen=True)
class SinusoidSpec:
    """Absolute position vector added to the embedding: entry 2i = sin(p * base^(-2i/dim)), entry
    2i+1 = cos of the same angle."""
    dim: int
    base: float = 10000.0


@dataclass(frozen=True)
class RotaryHalfSpec:
    """Rotate-half rotary encoding over the whole head: angle(p, j) = p * theta^(-2j/dim)."""
    dim: int
    theta: float


@dataclass(frozen=True)
class RotaryPartSpec:
    """Rotate-half rotation of the first ``dim`` coordinates of a head (coordinate i with i + dim/2, i below
    dim/2) by angle(p, i) = p * base^(-2i/dim); the head's other coordinates pass. The frequencies are made in
    float64 and rounded to float32 once; the angle is their float32 product with the position."""
    dim: int
    base: float


@dataclass(frozen=True)
class RotaryPairsSpec:
    """Rotation of neighbouring pairs over the first ``dim`` coordinates of a vector (coordinate 2i with 2i + 1, i below
    dim/2) by angle(p, i) = p * base^(-2i/dim); the other coordinates pass. Frequencies and angles as ``RotaryPartSpec``."""
    dim: int
    base: float


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query softmax attention with q/k/v/o projections without bias."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                               # multiplies q.k before the softmax
    qk_norm: Optional[Any] = None              # norm spec over head_dim applied to q and k heads
    position: Optional[Any] = None             # position-encoding spec applied to q and k
    window: Optional[int] = None               # keys a query sees, itself included; None: all


@dataclass(frozen=True)
class MaskedAttentionSpec:
    """Causal grouped-query softmax attention without rotation, with options: value heads of a size
    of their own; a chunk mask (position i sees j <= i only if floor(i / chunk) == floor(j / chunk),
    chunks counted from the sequence's first position) and/or a sliding window; a logarithmic distance
    bias taken off the score, r1_h * ln(1 + r2_h * (i - j)), with two learned numbers a head; a sink (a
    learned number a head whose exponential joins the softmax's denominator and nothing else); an
    output gate sigmoid(W_g x) on the concatenated heads before the output projection.
    Further options: ``keep_first`` (the first that many positions of a sequence stay in sight of every later
    query when the window has moved on, at their true positions); ``softcap`` (score <- cap * tanh(score /
    cap), after the scale and before the masks); ``unit_sink`` (a sink fixed at score 0, so the softmax's
    denominator is one plus the sum; no tensor); and what may stand between the projection and the cache:
    ``conv_taps`` (a causal convolution over time of that many taps on every channel of q, k and v, tensors
    ``<q|k|v>.conv`` [channels, taps], its memory a per-sequence state), ``qk_norm`` (a norm spec over
    head_dim for q and k heads, tensors ``q.norm`` / ``k.norm``; a ``UnitRMSNormSpec`` has no tensors) and ``position``
    (a ``RotaryPartSpec``); the norm comes before the rotation unless ``norm_after_rotation``.
    ``value_mix``: the layers of a model that say it share the values of the first of them ("source": it leaves its
    values of the step's tokens for the others and caches them as they are); every other ("blend") caches and uses
    v <- (1 - lam) v + lam v_source with its learned number ``vmix`` (both kinds hold the tensor; the source's is unused).
    ``values_in_keys``: a token's value row is the first ``v_head_dim`` numbers of its key row (the rows of latents of an
    attention through latents): the cache keeps the key rows alone and every kernel reads values from them (the tcgen05 prompt
    kernel and the split single-token kernel, which want a store of values, are not used then).
    ``bias``: q, k and v have biases (tensors ``q.b``, ``k.b``, ``v.b``), added in the projection. ``q_temp`` = (coef,
    every): q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1). ``talk``: the heads' scores are
    mixed before the masks and the softmax, score_h <- sum_g T[h, g] score_g with the tensor ``talk`` [heads, heads]."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    chunk: Optional[int] = None
    window: Optional[int] = None
    distance_bias: bool = False
    sink: bool = False
    output_gate: bool = False
    keep_first: int = 0
    softcap: Optional[float] = None
    unit_sink: bool = False
    conv_taps: Optional[int] = None
    qk_norm: Optional[Any] = None
    position: Optional[Any] = None
    norm_after_rotation: bool = False
    value_mix: Optional[str] = None
    values_in_keys: bool = False
    bias: bool = False
    q_temp: Optional[Tuple[float, int]] = None
    talk: bool = False


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention: every head has two softmax maps over the same values. q has heads * 2 * head_dim rows and
    k kv_heads * 2 * head_dim, head by head as [map 1 | map 2]; q, k, v have biases (``q.b`` ..); no rotation; q at
    position p times 1 + coef * ln(floor((p + 1) / every) + 1) with ``q_temp`` = (coef, every); each map is a causal
    softmax of (q . k) * scale (inside ``window`` if given). With a1, a2 the maps' outputs and lambda = exp(lq1 . lk1) -
    exp(lq2 . lk2) + diff (tensors of size head_dim), a head's output is unit_rms(a1 - lambda a2) * (1 - diff), the root
    mean square over its v_head_dim values with ``norm_eps`` inside the root; then the output projection ``o``."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    diff: float
    norm_eps: float
    q_temp: Optional[Tuple[float, int]] = None
    window: Optional[int] = None


@dataclass(frozen=True)
class LowerBoundRecurrenceSpec:
    """HGRN2: linear attention whose forget gate also decides what is written. q = silu(W_q x) (heads x head_dim), v =
    W_v x (heads x v_head_dim), f = l + (1 - l) sigmoid(W_f x + b) per head and channel with the lower bound l = ``lower``;
    per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T (state [head_dim, v_head_dim], float32, zero at the start), o_t =
    S_t^T q_t; each head's o through an RMS norm over v_head_dim with the weight ``norm`` shared by the heads; then ``o``."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    norm_eps: float


@dataclass(frozen=True)
class StateSpaceSpec:
    """Mamba-2 (state-space duality). inner = heads * v_head_dim, N = state_dim, G = groups. ``in`` x is laid out as
    [z: inner | x: inner | B: G N | C: G N | dt: heads]; x, B, C pass a causal convolution per channel (``conv`` [channels,
    taps], last column the current token's, bias ``conv.b``) and SiLU; dt <- softplus(dt + dt_bias); per head (head h
    reads group h / (heads / G)) S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T (state [N, v_head_dim], float32), y_t =
    S_t^T C_t + D_h x_t; y * silu(z), an RMS norm in ``norm_groups`` equal parts times ``norm``, then ``o``. The last
    taps - 1 inputs of the convolution are per-sequence state too."""
    hidden_size: int
    num_heads: int
    v_head_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose queries, keys and values come through low-rank latents. With x the mixer's input:
    c_q = norm(W_dq x) (weight ``dq.norm``), q = W_uq c_q laid out head by head as [head_dim plain | rot_dim rotated];
    W_dkv x has kv_rank + rot_dim rows: the first kv_rank, normed (weight ``dkv.norm``), are the latent c, the last
    rot_dim, rotated by ``position`` and not normed, are one key part all heads share. Per head the plain key is
    W_uk c and the value W_uv c; score = (q_plain . k_plain + q_rot . k_rot) * scale; causal, inside ``window`` and/or
    ``chunk``; softmax; output projection ``o`` on the concatenated heads. The cache holds c and the rotated key part only."""
    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    norm_eps: float
    position: Optional[Any] = None
    window: Optional[int] = None
    chunk: Optional[int] = None


@dataclass(frozen=True)
class LinearAttentionSpec:
    """Linear attention with a constant decay per head: q, k, v = silu(W x); per head
    S_t = decay_h * S_(t-1) + k_t v_t^T (state [head_dim, v_head_dim], float32, zero at the start),
    o_t = S_t^T q_t; all heads together through ``out_norm`` (a weighted RMS norm over
    num_heads * v_head_dim), times sigmoid(W_g x) when ``output_gate``, then the output projection."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    decay: Tuple[float, ...]
    out_norm: Any = None
    output_gate: bool = True


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a decay per key channel and token: q = W_q x * head_dim^(-1/2), k = W_k x,
    v = W_v x; alpha = sigmoid(W_a2 (W_a1 x) + b)^(1/tau) laid out heads x head_dim (``decay_rank`` the inner
    size of the two-step projection); per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T (state
    [head_dim, v_head_dim], float32, zero at the start), o_t = S_t^T q_t; each head's o through an RMS norm
    over v_head_dim with one weight shared by the heads, times silu(W_g x), then the output projection."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    decay_rank: int
    tau: float
    norm_eps: float


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input; the result is the sum of scale_i * mixer_i(x).
    ``branches``: (checkpoint prefix under the mixer, mixer spec, scale) each."""
    hidden_size: int
    branches: Tuple[Tuple[str, Any, float], ...]


@dataclass(frozen=True)
class DenseMLPSpec:
    """down(act(up(x))) without bias. ``activation`` "xielu": with two learned numbers p, q,
    act(z) = softplus(p) z^2 + z/2 for z > 0 and (1/2 + softplus(q)) (e^z - 1 - z) + z/2 otherwise."""
    hidden_size: int
    intermediate_size: int
    activation: str = "xielu"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) without bias; ``activation`` "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi)
    (z + 0.044715 z^3)))). ``names``: the tensors' names under the part's prefix (gate, up, down)."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of experts: ``num_experts`` gated feed-forwards (tensors ``e<i>.gate/up/down``, inner size
    ``expert_ff``) of which a token uses ``top``. Router: s = sigmoid(W_router x) in float32; the choice goes by
    s + ``correction`` (a tensor), among the experts of the ``keep_groups`` best of ``groups`` equal groups of
    neighbours (group score: the sum of its two largest choice scores), the ``top`` largest; the weights are the
    chosen s over their sum (+ 1e-20), times ``route_scale``. ``shared_ff``: a shared expert of that inner size
    (``shared.gate/up/down``) runs for every token, times sigmoid(w_sg . x) (``shared.sg`` [1, hidden]).
    Options: ``correction`` False: no such tensor, the choice goes by s; ``renorm`` False: the weights are the chosen s
    themselves (times ``route_scale``); ``weight_on_input``: the weight multiplies the expert's input, out = sum
    expert(w x), not its output; ``shared_gate`` False: the shared expert is added as it is. ``activation`` "clamped":
    with g = min(gate x, limit), u = clamp(up x, -limit, limit) an expert is down(g sigmoid(1.702 g) (u + 1)), with
    ``limit`` for the routed experts and ``shared_limit`` for the shared one."""
    hidden_size: int
    expert_ff: int
    num_experts: int
    top: int
    groups: int = 1
    keep_groups: int = 1
    route_scale: float = 1.0
    shared_ff: Optional[int] = None
    activation: str = "silu"
    correction: bool = True
    renorm: bool = True
    weight_on_input: bool = False
    shared_gate: bool = True
    limit: Optional[float] = None
    shared_limit: Optional[float] = None


@dataclass(frozen=True)
class LayerSpec:
    """One pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).
    ``prefix`` is the layer's tensor-name prefix in the checkpoint. A layer without a feed-forward has
    ``norm_post`` and ``feed_forward`` None (and no names for them)."""
    prefix: str
    norm_in: Any
    mixer: Any
    norm_post: Any
    feed_forward: Any
    # checkpoint name of each sub-part under the prefix
    names: Tuple[Tuple[str, str], ...] = (("norm_in", "input_layernorm."), ("mixer", "self_attn."),
                                          ("norm_post", "post_attention_layernorm."), ("feed_forward", "mlp."))


@dataclass(frozen=True)
class PostNormLayerSpec:
    """One block with the norm after the sum: x <- norm_mix(alpha * x + mixer(x)), then
    x <- norm_ff(alpha * x + feed_forward(x)); the sublayers read x itself. Without a feed-forward the second
    step, its norm and their names fall away."""
    prefix: str
    mixer: Any
    norm_mix: Any
    feed_forward: Any
    norm_ff: Any
    alpha: float = 1.0
    names: Tuple[Tuple[str, str], ...] = (("mixer", "mix."), ("norm_mix", "norm1"), ("feed_forward", "mlp."),
                                          ("norm_ff", "norm2"))


@dataclass(frozen=True)
class SandwichLayerSpec:
    """One block with a norm before and after each sublayer: x <- x + norm_mix_out(mixer(norm_in(x))), then
    x <- x + norm_ff_out(feed_forward(norm_post(x))). Without a feed-forward the second step, its norms and their names
    fall away."""
    prefix: str
    norm_in: Any
    mixer: Any
    norm_mix_out: Any
    norm_post: Any
    feed_forward: Any
    norm_ff_out: Any
    names: Tuple[Tuple[str, str], ...] = (("norm_in", "norm1."), ("mixer", "mix."), ("norm_mix_out", "norm1b."),
                                          ("norm_post", "norm2."), ("feed_forward", "mlp."), ("norm_ff_out", "norm2b."))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` names the cache entry the layer's mixer uses; with
    ``writes=False`` the mixer only reads what the entry's owner stored in this step. Right before the
    run the residual stream may take in the embedding's output once more (``add_embedding``) and a row
    of a learned table of the model (``add_row`` = (name in ``ModelSpec.tables``, row))."""
    layer: int
    cache: int
    writes: bool = True
    add_embedding: bool = False
    add_row: Optional[Tuple[str, int]] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_embeddings: Optional[bool]             # None: decided by the checkpoint (lm_head present or not)
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    embed_scale: float = 1.0                   # multiplies the embedding row
    embed_position: Optional[Any] = None       # position spec whose vector is added to the embedding
    logit_cap: Optional[float] = None          # logits <- cap * tanh(logits / cap)
    logit_scale: float = 1.0                   # multiplies the logits before the cap
    tables: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()   # learned float32 tables of the model itself: (checkpoint name, shape)
    unused_tensors: Tuple[str, ...] = ()       # checkpoint names the design ships although nothing reads them
    extra: dict = field(default_factory=dict, compare=False)

    @staticmethod
    def identity_schedule(n_layers):
        return tuple(ScheduleEntry(i, i, True) for i in range(n_layers))
