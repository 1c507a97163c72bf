"""Declarative description of a decoder: what each part is and how layers are arranged.

An architecture turns its typed configuration into one ``ModelSpec``. Every size
and constant a part needs is a field of its spec, so no part knows which model it
is in; ``kind`` selects the implementation from the part registries, layer by
layer, so one model may mix different mixers and feed-forwards. The order in
which layers run is data as well (``run_order``): an entry may name a layer twice
or let a layer read another layer's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One checkpoint tensor a part wants.

    role: 'matrix' and 'table' are kept in the engine dtype (bfloat16 or float32),
    'vector' is always float32 (biases, norm parameters), 'int' is int32.
    ``stored_in_out``: the checkpoint holds the matrix as [in, out] (GPT-2 Conv1D);
    the device copy is always [out, in], K-contiguous.
    ``pieces``: the checkpoint does not hold this tensor whole but as several tensors
    ((checkpoint name, shape as stored), ...) that are joined along the output axis, in
    this order, when they are placed (separate query, key and value projections that one
    fused product reads); ``name`` is then only the key under which the part finds the
    joined tensor, and ``shape`` its shape as if it had been stored whole.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    stored_in_out: bool = False
    pieces: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()


@dataclass(frozen=True)
class NormSpec:
    kind: str            # 'layernorm' | 'rmsnorm' | 'tanh' (tanh(alpha x) * weight + bias: no statistics, eps unused)
    width: int
    eps: float
    weight: str          # checkpoint names
    bias: Optional[str] = None
    weight_offset: float = 0.0   # 'rmsnorm': the factor is weight_offset + weight (1 for a weight stored around zero)
    groups: int = 1              # 'rmsnorm': the row in this many equal consecutive stretches, each divided by its own
                                 # root mean square (the weight spans the whole row)
    alpha: Optional[str] = None  # 'tanh': checkpoint name of the one number that multiplies x inside the tanh


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # 'learned'
    n_positions: int
    width: int
    table: Optional[str] = None


@dataclass(frozen=True)
class LongContextBlend:
    """Rotary frequencies blended for contexts beyond the one a model was trained at (the YaRN rule): pair i keeps
    its frequency f_i where its wavelength turns more than ``fast`` times over ``original`` tokens, gets f_i / factor
    where it turns fewer than ``slow`` times, a linear blend between; cosine and sine are scaled by
    0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class WavelengthStretch:
    """Rotary frequencies stretched for contexts beyond the one a model was trained at, by wavelength l = 2 pi / f: a pair
    keeps f where l < original / high, gets f / factor where l > original / low, and between the two, with
    s = (original / l - low) / (high - low), (1 - s) f / factor + s f. Cosine and sine are not scaled."""
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class RotarySpec:
    kind: str            # 'rotary'
    head_dim: int
    dims: int            # the first `dims` dimensions of a head are rotated, the rest pass unchanged
    base: float
    interleaved: bool = True     # pairs are neighbours (2i, 2i+1); False: halves (i, i + dims/2)
    blend: object = None         # None, a LongContextBlend or a WavelengthStretch


@dataclass(frozen=True)
class AttentionSpec:
    kind: str            # 'attention'
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float         # multiplies q.k (already includes any per-layer factor)
    window: Optional[int]  # None = all earlier keys; n = the query and the n-1 keys before it
    qkv_weight: object   # checkpoint name of the fused projection, or the three names (query, key, value) of separate ones
    qkv_bias: object     # None, one name, or three names
    out_weight: str
    out_bias: Optional[str]
    stored_in_out: bool = False
    value_dim: Optional[int] = None   # size of a value head where it differs from head_dim
    chunk: Optional[int] = None       # positions in chunks of this many from the start; nothing is seen across a border
    gate_weight: Optional[str] = None  # [n_heads, width]: a head's output is multiplied by sigmoid(gate . input)
    rotary: object = None             # a position-encoding spec of the mixer's own (applied to its queries and keys)
    # RMS norm of every query head and every key head over the head's dimensions, before the rotation: the checkpoint
    # names of the two weights [head_dim] (one weight for all heads of a kind; None for a kind that is not normed)
    query_norm: Optional[str] = None
    key_norm: Optional[str] = None
    head_norm_eps: float = 1e-6
    # False: the mixer has no key and value projections (qkv_weight names the query projection alone) and reads
    # the cache of another stop of the run order (RunEntry.cache_of), with its own queries, mask and scale
    own_keys_values: bool = True
    # keys kept in the cache where other stops read it through a wider mask than this mixer's own ('all': every key);
    # None: what the mixer's own window needs
    keep_window: object = None
    # behind a window, the first so many keys of the sequence stay visible (at their true positions)
    keep_first: int = 0
    # c: a scaled score s becomes c * tanh(s / c)
    softcap: Optional[float] = None
    # checkpoint name of one number per head, [n_heads]: exp(sink) joins the softmax's denominator (a key without a
    # value; it is neither scaled nor capped)
    sink: Optional[str] = None
    # values blended over layers: a mixer with value_mix_source leaves its values of the step's tokens for later mixers;
    # one with value_mix (the checkpoint name of a single number w) replaces its values by (1 - w) v + w * those, before
    # they are cached
    value_mix_source: bool = False
    value_mix: Optional[str] = None
    # the softmax weights meet the values unrounded: a tensor-core kernel splits each into two bfloat16 terms instead of
    # rounding it to one (the float32 kernels do so anyway)
    exact_weights: bool = False
    # the values are the keys as projected, before their norm and rotation: the mixer has no value projection (qkv_weight
    # names the query and key projections only; value_dim must be head_dim)
    values_are_keys: bool = False
    # the norm of queries and of keys runs over the whole projection (all heads at once) instead of over every head;
    # query_norm and key_norm then name weights [n_heads * head_dim] and [n_kv_heads * head_dim]
    norm_whole_projection: bool = False
    # the gate (gate_weight) has a row per element of the attended output, [n_heads * value_dim, width], instead of one per head
    gate_per_element: bool = False
    # one is added to the softmax's denominator (a sink whose score is 0 and that needs no tensor)
    unit_sink: bool = False


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are projections of one small latent row per token. q = W_q y, per head
    [head_dim plain | rot_dim rotated]. W_down y = [rank | rot_dim]: the first part, RMS-normed with ``latent_norm``
    (eps ``norm_eps``), is the latent c; the second, rotated, is a key part all heads share. Per head the plain key is
    W_up_key c and the value W_up_value c; score = (q_plain . k_plain + q_rot . k_rot) * scale over every earlier token;
    ``sink`` as in ``AttentionSpec``. Only c and the rotated key part are cached."""
    kind: str            # 'latent_attention'
    width: int
    n_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    rank: int
    scale: float
    norm_eps: float
    rotary: object       # a RotarySpec over the rot_dim part (head_dim = rot_dim there)
    query_weight: str    # checkpoint names; matrices [out, in]
    down_weight: str
    latent_norm: str
    up_key_weight: str
    up_value_weight: str
    out_weight: str
    sink: Optional[str] = None


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule with a decay per key channel. q = W_q y, k = W_k y ([n_kv_heads, head_dim]), v = W_v y
    ([n_heads, value_dim]); each passes a short causal convolution over time per channel (``conv_taps`` taps, weights
    '<projection>.conv' [channels, taps], the last tap is the current token's) and silu; q and k become unit vectors
    per head (x / sqrt(sum x^2 + 1e-6)), q times head_dim^-1/2; head h uses q/k head h // (n_heads / n_kv_heads).
    beta = sigmoid(W_beta y) per head; decay = exp(-exp(A_log[head]) * softplus(W_a2 (W_a1 y) + dt_bias)) per head and
    key channel. Per head S <- decay[:, None] * S; u = beta * (v - S^T k); S <- S + k u^T; o = S^T q, S float32 per
    request from zero. o is divided by its root mean square per head (``norm_eps``), multiplied by ``out_norm`` [value_dim]
    and by sigmoid(W_g2 (W_g1 y)), and projected by W_out."""
    kind: str            # 'gated_delta'
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    norm_eps: float
    query_weight: str    # checkpoint names; matrices [out, in]
    key_weight: str
    value_weight: str
    beta_weight: str
    decay_down: str
    decay_up: str
    decay_log: str       # A_log [n_heads]
    decay_bias: str      # dt_bias [n_heads * head_dim]
    gate_down: str
    gate_up: str
    out_norm: str
    out_weight: str


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head and no softmax: per head S_t = decay * S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t, the state S [head_dim, value_dim] float32 per request, from zero. Queries and keys may be rotated
    (``rotary``); keys are multiplied by ``key_scale`` after the rotation. Every head's o is divided by its root mean
    square (``norm_eps`` inside the root, no weight), multiplied by silu(W_gate y) and projected by W_out."""
    kind: str            # 'retention'
    width: int
    n_heads: int
    head_dim: int
    value_dim: int
    decay: Tuple[float, ...]       # one per head
    key_scale: float
    norm_eps: float
    query_weight: str    # checkpoint names; matrices [out, in]
    key_weight: str
    value_weight: str
    gate_weight: str
    out_weight: str
    rotary: object = None


@dataclass(frozen=True)
class StateSpaceSpec:
    """A state-space mixer with a scalar decay per head. W_in y = [z: inner | x: inner | B: groups * state | C: groups * state
    | dt: n_heads] with inner = n_heads * value_dim; x, B and C together pass a short causal convolution per channel
    (``conv_weight`` [channels, conv_taps], the last tap is the current token's, bias ``conv_bias``) and silu;
    dt = softplus(dt + dt_bias). Per head h (group h // (n_heads / groups)), S [state, value_dim] float32 per request from
    zero: S <- exp(-exp(A_log[h]) dt) S + dt B x^T, y = S^T C + D[h] x. y * silu(z) is divided, in ``norm_groups`` equal
    stretches, by its root mean square (``norm_eps``), multiplied by ``out_norm`` [inner] and projected by W_out."""
    kind: str            # 'state_space'
    width: int
    n_heads: int
    value_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    in_weight: str       # checkpoint names; matrices [out, in]
    conv_weight: str
    conv_bias: str
    dt_bias: str
    decay_log: str       # A_log [n_heads]
    skip: str            # D [n_heads]
    out_norm: str
    out_weight: str


@dataclass(frozen=True)
class LinearRecurrenceSpec:
    """A gated linear recurrence per channel. Two branches of ``inner`` channels: g = gelu_tanh(W_gate y + b) and
    u = conv(W_in y + b), a short causal convolution per channel with a bias and no activation. The channels come in
    ``blocks`` equal parts; in part p, r = sigmoid(Ra[p] u_p + ba[p]) and i = sigmoid(Ri[p] u_p + bi[p]);
    a = exp(-gain * r * softplus(lam)); S <- a S + sqrt(1 - a^2) i u per channel, float32 per request from zero; the output
    is W_out (S * g)."""
    kind: str            # 'linear_recurrence'
    width: int
    inner: int
    blocks: int
    conv_taps: int
    gain: float
    gate_weight: str     # checkpoint names; matrices [out, in]
    gate_bias: str
    in_weight: str
    in_bias: str
    conv_weight: str
    conv_bias: str
    decay_gate: str      # Ra [blocks, part, part]
    decay_gate_bias: str
    input_gate: str      # Ri
    input_gate_bias: str
    decay_param: str     # lam [inner]
    out_weight: str


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is ``factor`` * (norm(left) * left_norm + norm(right) * right_norm),
    each output divided by its root mean square over the model width (``norm_eps``) and multiplied by its weight [width]."""
    kind: str            # 'side_by_side'
    width: int
    left: object         # mixer specs
    right: object
    left_norm: str       # checkpoint names
    right_norm: str
    norm_eps: float
    factor: float = 0.5


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str            # 'dense'
    width: int
    inner: int
    activation: str      # 'gelu_new' | 'gelu' | 'relu2'
    up_weight: str
    up_bias: Optional[str]
    down_weight: str
    down_bias: Optional[str]
    stored_in_out: bool = False


@dataclass(frozen=True)
class GatedUnitSpec:
    """A small feed-forward of three matrices, W_down (f(W_gate y, W_up y)), no biases. ``activation``:
    'clamped_swish'  g = min(gate, limit), u = clamp(up, -limit, limit), f = g * sigmoid(alpha g) * (u + 1);
    'silu'           f = gate * sigmoid(gate) * up;
    'gelu_tanh'      f = 0.5 gate (1 + tanh(sqrt(2/pi) (gate + 0.044715 gate^3))) * up
    (limit and alpha belong to the first only)."""
    inner: int
    limit: float
    gate_weight: str
    up_weight: str
    down_weight: str
    alpha: float = 1.702
    activation: str = "clamped_swish"


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """A dense feed-forward that is one gated unit: residual + W_down (f(W_gate y, W_up y))."""
    kind: str            # 'gated'
    width: int
    unit: GatedUnitSpec

    @property
    def inner(self):
        return self.unit.inner


@dataclass(frozen=True)
class TableRoutedExpertsSpec:
    kind: str            # 'experts_by_table'
    width: int
    vocab_size: int
    top: int             # experts per token; each weighs 1 / top
    table: str           # checkpoint name of the integer table [vocab, top]: a token id's experts
    experts: Tuple[GatedUnitSpec, ...]       # all of one size and limit
    shared: Optional[GatedUnitSpec] = None   # runs for every token and is added


@dataclass(frozen=True)
class ScoreRoutedExpertsSpec:
    """Experts chosen per token by a router: z = W_router y in float32, s = ``score``(z) ('sigmoid'); the experts
    form ``groups`` equal runs of neighbours, a run's worth is the sum of its two largest scores, only experts of the
    ``keep_groups`` worthiest runs can be chosen; the ``top`` largest eligible scores win. A chosen expert's output is
    weighted by s * weight_scale (not renormalised). ``shared``: a unit that runs for every token; with
    ``shared_gate`` (a checkpoint name, [1, width]) its output is multiplied by sigmoid(gate . y)."""
    kind: str            # 'experts_by_score'
    width: int
    top: int
    router: str          # checkpoint name of W_router [experts, width]
    experts: Tuple[GatedUnitSpec, ...]       # all of one size and activation
    groups: int = 1
    keep_groups: int = 1
    weight_scale: float = 1.0
    score: str = "sigmoid"
    shared: Optional[GatedUnitSpec] = None
    shared_gate: Optional[str] = None


@dataclass(frozen=True)
class NoFeedForwardSpec:
    kind: str = "none"


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a mixer, a feed-forward, as many norms as its arrangement wants, and the arrangement that wires them
    ('pre_norm' takes two norms: before the mixer, before the feed-forward; 'pre_norm_mixer' one norm and no
    feed-forward; 'parallel' one norm whose output both the mixer and the feed-forward read; 'pre_norm_shift' is
    'pre_norm', or 'pre_norm_mixer' with one norm, whose mixer reads its normed input blended per channel with the
    normed input of the token before: n[t] + (n[t-1] - n[t]) * ``shift_weight`` [width], n[-1] = 0)."""
    arrangement: str
    mixer: object
    feed_forward: object
    norms: Tuple[object, ...]
    shift_weight: Optional[str] = None

    @property
    def kind(self):
        return self.arrangement


@dataclass(frozen=True)
class EmbeddingSpec:
    kind: str            # 'tokens': a row of the table per token id (the position encoding may add its own table)
    vocab_size: int
    width: int
    table: str           # checkpoint name
    scale: float = 1.0   # multiplies the row


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """A row of the token table plus a row of a table of token pairs: row (previous id * mul_prev + id * mul_cur) mod buckets
    of ``pair_table`` [buckets + 1, width]; a sequence's first token takes the last row. The id before a step's first token
    is kept per request."""
    kind: str            # 'tokens_pairs'
    vocab_size: int
    width: int
    table: str           # checkpoint names
    pair_table: str
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class HeadSpec:
    kind: str            # 'linear': final norm on the wanted rows, then logits = y . W^T (+ bias)
    vocab_size: int
    width: int
    norm: object         # a norm spec
    weight: str          # checkpoint name of W [vocab, width]
    tied: bool = False   # W is the embedding's table (declared there, not again)
    bias: Optional[str] = None
    softcap: Optional[float] = None   # c: logits become c * tanh(logits / c)


@dataclass(frozen=True)
class RunEntry:
    """One stop of the forward pass: run ``layer`` (an index into ``ModelSpec.layers``).

    Every stop has a cache of its own, so a layer that is named twice keeps the keys and
    values of its two runs apart. ``cache_of`` = the index of an EARLIER STOP in
    ``run_order`` makes this stop read that stop's cache instead: it gets no pages of its
    own and does not write (its mixer sees ``cache.writable == False``).
    """
    layer: int
    cache_of: Optional[int] = None
    # before the stop runs (the start of a repeated pass over a run of layers): the embedding's output is added to the
    # stream, and/or row ``add_vector`` of the model's ``pass_vectors`` table
    add_embedding: bool = False
    add_vector: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: Optional[int]      # None: the architecture sets no limit (the engine's cache does)
    embedding: object                 # an embedding spec
    position: object                  # a position-encoding spec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    head: object                      # a head spec (with the final norm)
    # Streams mixed over depth: None, or per stop of the run order the checkpoint name of its weights [stop + 2]. With
    # X_0 the embedding's output and X_(i+1) what stop i leaves, what stop i + 1 (and after the last stop the head)
    # reads is sum over j <= i + 1 of weights_i[j] * X_j
    depth_mix: Optional[Tuple[str, ...]] = None
    # (checkpoint name, rows) of a float32 table [rows, width] whose rows stops of the run order add to the stream
    # (RunEntry.add_vector)
    pass_vectors: Optional[Tuple[str, int]] = None
    eos_token_ids: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)   # regexes of tensors to drop
    tied_duplicates: Tuple[Tuple[str, str], ...] = field(default_factory=tuple)  # (name, must equal)
    optional_prefix: str = ""          # e.g. 'transformer.': stripped from every name when present

    @property
    def prefix_probe(self):
        """The tensor whose presence under the optional prefix says that the checkpoint uses the prefix."""
        return self.embedding.table
