"""Architecture-neutral description of a decoder: what the parts are and how they are arranged.

A model is data: an embedding, a list of layers, a schedule that says in which order the layers
run (and whose cache each run uses), a final norm and a head.  Every layer names its parts by
*kind* and carries the sizes and constants of each part; nothing here knows which architecture it
describes.  An architecture (see ``gophonic_b200.registry``) is a function from its own typed
configuration to a ``ModelSpec``.

The reference keeps the same information in one flat ``modelConfig`` with per-layer flags
(internal/qwen3lm/weights.go:108-127, the ``linear []bool`` per-layer kind list at :122); here it
is split per part so that a new mixer or feed-forward is a new spec class, not a new field on a
shared struct.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (offset + weight)  (internal/qwen3lm/ops.go:251-254).  The
    weight is the tensor ``prefix + tensor``; with ``offset`` 1 the checkpoint holds the weight's difference from one.
    ``gain`` multiplies the normed row once more (a model that scales its logits by a constant gives that
    constant to its final norm: the head is linear)."""
    size: int
    eps: float
    kind: str = "rmsnorm"
    tensor: str = "weight"
    offset: float = 0.0
    gain: float = 1.0     # one more factor on the output, folded into the weight when it is loaded: (offset + weight) * gain


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary embedding over the first ``rotary_dim`` elements of each head.

    inv_freq_i = theta^(-2i/rotary_dim) (internal/qwen3lm/weights.go:681-688); element i pairs with
    i + rotary_dim/2 (internal/qwen3lm/kernels_scalar.go:73-80).

    ``scaling`` = (factor, low, high, original) stretches the slow frequencies for contexts longer than
    ``original`` positions: a frequency f whose wavelength 2 pi / f is longer than original / low becomes
    f / factor, one whose wavelength is shorter than original / high stays, and in between
    s = (original / wavelength - low) / (high - low) blends them as (1 - s) f / factor + s f.
    """
    head_dim: int
    rotary_dim: int
    theta: float
    kind: str = "rope"
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class PairRotarySpec:
    """Rotary embedding in which neighbouring channels turn together: channels 2i and 2i + 1 of a
    head, i < rotary_dim / 2, by the angle pos * theta^(-2i/rotary_dim); the channels from
    ``rotary_dim`` on pass unchanged.  ``scaling`` as for ``RotarySpec``."""
    head_dim: int
    rotary_dim: int
    theta: float
    kind: str = "rope_pairs"
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    head_dim: int
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention (internal/qwen3lm/ops.go:231-293).

    ``qk_norm`` is the per-head norm applied to q and k before the position encoding, or None.
    ``window`` = 0 attends to every earlier key; w > 0 only to the last w keys (itself included).
    """
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    scale: float
    position: object
    qk_norm: Optional[RMSNormSpec] = None
    window: int = 0
    kind: str = "attention"


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Grouped-query attention with the options of the Pugalix design, each of which can be left off:

    * ``bias``: q, k and v projections carry a bias;
    * ``value_dim``: a value head may have another size than a query/key head;
    * ``window`` > 0 with ``keep_first``: position i sees j <= i if i - j < window or j < keep_first;
    * ``sink``: the softmax denominator carries one more unit, p_j = exp(s_j) / (1 + sum exp(s)); with
      ``sink_learned`` the unit is exp(z_h) instead, z_h one learned number per head (tensor ``sink``), which
      is not scaled and has no key and no value;
    * ``qk_norm`` (an ``RMSNormSpec`` whose eps is used): q and k are RMS-normed after their biases and before the
      position encoding; with ``qk_norm_span`` over the whole projection at once (all heads of q share one mean of
      squares and a weight of heads * head_dim, tensor ``q.norm``; k likewise), else head by head with a weight
      of head_dim;
    * ``out_bias``: the output projection carries a bias too;
    * ``gate``: the concatenated heads are multiplied by sigmoid of a further projection of the
      mixer's input before the output projection;
    * ``own_kv`` False: the layer has no key/value projections and reads the cache plane of an
      earlier run (``ScheduleEntry.cache_of``), with queries, mask and the rest of its own.

    ``names`` maps q, k, v, g, o to tensor-name suffixes under the mixer's prefix; a bias is the
    projection's name plus ``bias_suffix``."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: object
    window: int = 0
    keep_first: int = 0
    sink: bool = False
    bias: bool = False
    gate: bool = False
    own_kv: bool = True
    sink_learned: bool = False
    qk_norm: Optional[RMSNormSpec] = None
    qk_norm_span: bool = False
    out_bias: bool = False
    names: Tuple[Tuple[str, str], ...] = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q_norm", "q.norm"),
                                          ("k_norm", "k.norm"), ("sink", "sink"))
    bias_suffix: str = ".b"
    kind: str = "gated_attention"


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention: every query head has two softmax maps over the same values and its output is the first
    less ``lambda`` times the second.  q holds heads * 2 * head_dim rows and k kv_heads * 2 * head_dim, head by head
    as [map 1, map 2]; v holds kv_heads * value_dim; query head h reads key/value head h // (heads / kv_heads).
    Per head and map q and k are RMS-normed over ``head_dim`` (``qk_norm``, one weight of head_dim for q and one for k)
    and then given the position encoding.  Scores (q . k) * scale over the keys j <= i that the mask leaves:
    ``chunk`` > 0: only those in i's own block of ``chunk`` positions, counted from the sequence's start; ``window`` > 0:
    only those with i - j < window.  With

        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init        (four learned vectors of head_dim)

    head h's output is o = a1 - lambda a2, o / sqrt(mean(o^2) + eps) * (1 - lambda_init), and the heads go
    through the output projection.  ``names`` maps q, k, v, o, the two norms and the four vectors to tensor-name
    suffixes under the mixer's prefix."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: object
    lambda_init: float
    eps: float
    qk_norm: Optional[RMSNormSpec] = None
    chunk: int = 0
    window: int = 0
    names: Tuple[Tuple[str, str], ...] = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                                          ("lq1", "lq1"), ("lk1", "lk1"), ("lq2", "lq2"), ("lk2", "lk2"))
    kind: str = "diff_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose queries, keys and values are made from low-rank latents.  With h the mixer's input:

        c_q = rmsnorm(W_dq h) (q_rank, weight ``dq.norm``),   q = W_uq c_q: per head [head_dim plain | rot_dim rotated]
        W_dkv h = [kv_rank | rot_dim]:  c = rmsnorm(first part) (weight ``dkv.norm``),  k_r = the rest, rotated, one for all heads
        per head: k = [W_uk c | k_r],  v = W_uv c  (value_dim),   score = (q . k) * scale

    Only c and k_r are cached.  ``position`` is the encoding of the rotated part (its ``head_dim`` is rot_dim);
    ``window`` > 0: row i sees j with 0 <= i - j < window; ``chunk`` > 0: only its own block of positions."""
    hidden: int
    heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    position: object
    eps: float
    window: int = 0
    chunk: int = 0
    names: Tuple[Tuple[str, str], ...] = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                                          ("uk", "uk"), ("uv", "uv"), ("o", "o"))
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DecayStateSpec:
    """Gated linear attention: per head a matrix state S (key_dim x value_dim, float32) with a decay
    per key channel, S <- diag(a) S + k v^T, o = S^T q, q scaled by key_dim^(-1/2).  The decay is
    a = sigmoid(W2 (W1 x) + b)^(1 / tau) with W1 of ``rank`` rows.  Each head's o is RMS-normed with
    one weight of ``value_dim`` shared by the heads, multiplied by silu of a gate projection, and
    projected back."""
    hidden: int
    heads: int
    key_dim: int
    value_dim: int
    rank: int
    tau: float
    eps: float
    kind: str = "gla"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """The matrix memory of an mLSTM: per head S (key_dim x value_dim), a normaliser n (key_dim) and a
    running maximum m, all float32 and zero at the start.  With log gates i = cap tanh(x_i / cap) and
    f = logsigmoid(cap tanh(x_f / cap)): m' = max(f + m, i), S <- exp(f + m - m') S + exp(i - m') k v^T,
    n likewise with k alone, o = S^T q / (max(|n . q|, exp(-m')) + 1e-6), q scaled by key_dim^(-1/2).
    Each head's o is divided by its root mean square; the heads together are multiplied by a weight
    and by sigmoid of a gate projection, and projected back."""
    hidden: int
    heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    kind: str = "mlstm"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Generalized delta rule: per head a matrix state S (key_dim x value_dim, float32).  With the
    receptance r, key k, value v, a decay w and a removal rate a per key channel and the unit key
    u = k / sqrt(|k|^2 + key_eps):

        S <- diag(w) S - (a * u) (u^T S) + k v^T   (both terms read the old S),   o = S^T r.

    w = exp(-decay_scale * sigmoid(W2 tanh(W1 x) + w0)) with W1 of ``rank`` rows (None: the
    checkpoint's), a = sigmoid(Wa x + b).  Each head's o is divided by its root mean square, the
    heads together are multiplied by a weight and by sigmoid of a gate projection, and projected back."""
    hidden: int
    heads: int
    key_dim: int
    value_dim: int
    rank: Optional[int]
    decay_scale: float
    key_eps: float
    eps: float
    kind: str = "delta_rule"


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    """Grouped-query attention whose weights are not normalised over the keys: a visible key j weighs
    sigmoid((q_i . k_j) * scale + b_h), with b_h one number per head (``score_bias``).  Options:

    * ``conv_taps`` > 0: a causal convolution over time on every channel of q, k and v directly after
      the projection, y_t = sum_j c[:, j] u_(t - taps + 1 + j), zeros before the sequence's start; the
      last taps - 1 projected rows of a sequence are part of its state;
    * ``qk_norm``: q and k are divided by their root mean square per head; ``v_norm``: v likewise (the
      cache holds the normed keys and values);
    * ``window`` > 0: position i sees j with 0 <= i - j < window; 0: every j <= i;
    * ``head_gate``: head h's output is multiplied by sigmoid of one number, row h of a further
      projection of the mixer's input.

    There is no position encoding."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: int = 0
    conv_taps: int = 0
    qk_norm: bool = True
    v_norm: bool = True
    score_bias: bool = True
    head_gate: bool = True
    eps: float = 1e-6
    kind: str = "sigmoid_attention"


@dataclass(frozen=True)
class MoESpec:
    """Mixture of experts: ``experts`` feed-forwards down(act(up(x))) without biases, act(z) = relu(z)^2,
    of which a token uses ``top``.  Router scores s = softmax(Wr x) over all experts in float32; the
    ``top`` largest are chosen and weigh their experts' outputs by s / (sum of the chosen s + renorm_eps).

    Each of these can be the other way:

    * ``score`` "sigmoid": s = sigmoid(Wr x), every expert's score by itself;
    * ``renorm`` False: the chosen scores are the weights as they are;
    * ``weight_on`` "input": a weight multiplies its expert's input, out = sum expert(w x), not its output;
    * ``act`` "swiglu": an expert is down(silu(gate x) * (up x)) with a third matrix ``e<j>.gate``;
    * ``act`` "glu_clamp": the same three matrices, down(g sigmoid(act_slope g) (u + 1)) with g = min(gate x, act_limit)
      and u = clamp(up x, -act_limit, act_limit);
    * ``shared``: the spec of a further feed-forward under ``shared_prefix`` that every token uses, with weight 1, or
      with ``shared_gate`` with weight sigmoid(w . x), w the tensor ``shared_prefix + shared_gate_name`` ([1, hidden]);
    * ``router_bias``: the router's logits carry a bias (tensor ``router`` + ``router_bias_suffix``);
    * ``renorm_eps`` 0 with ``score`` "softmax" and ``renorm``: the weights are the softmax over the chosen logits alone."""
    hidden: int
    experts: int
    top: int
    intermediate: int
    renorm_eps: float = 1e-20
    kind: str = "moe"
    score: str = "softmax"
    renorm: bool = True
    weight_on: str = "output"
    act: str = "relu2"
    shared: Optional[object] = None
    shared_prefix: str = "shared."
    act_limit: float = 0.0
    act_slope: float = 1.0
    router_bias: bool = False
    router_bias_suffix: str = ".b"
    shared_gate: bool = False
    shared_gate_name: str = "sg"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate(x)) * up(x))  (internal/qwen3lm/ops.go:442-461).  ``names``: the tensors of the
    gate, up and down projections under the part's prefix."""
    hidden: int
    intermediate: int
    kind: str = "swiglu"
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class ReluSquaredSpec:
    """down(relu(up(x))^2).  ``names``: the tensors of the up and down projections under the part's prefix."""
    hidden: int
    intermediate: int
    kind: str = "relu2_ff"
    names: Tuple[str, str] = ("up", "down")


@dataclass(frozen=True)
class ClampedGLUSpec:
    """down(g sigmoid(slope g) (u + 1)) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit)."""
    hidden: int
    intermediate: int
    limit: float
    slope: float
    kind: str = "glu_clamp"
    names: Tuple[str, str, str] = ("gate", "up", "down")


@dataclass(frozen=True)
class LayerSpec:
    """One layer of the pre-norm arrangement: the block kind and the four parts it arranges.

    ``prefix`` is the tensor-name prefix of the layer ("model.layers.3."); each part resolves its
    tensors under the sub-prefix named here (the defaults are the names Qwen3 checkpoints use).

    The model, the loader and the cache read only two fields of a layer's spec, ``block`` and
    ``prefix``; everything else is between the spec and the block class registered under that
    kind (``declare``, ``cache_request``, ``mixers``, ``prepare``, ``weight_bytes``, ``forward``).
    A block with another arrangement (one shared norm, norms after the parts, two mixers) brings a
    spec class of its own with those two fields.  ``feed_forward`` and ``feed_forward_norm`` None:
    the layer is its mixer sublayer alone.
    """
    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    block: str = "prenorm"
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class HyperLayerSpec:
    """One layer of the hyper-connection arrangement: the residual is ``streams`` copies x_1 .. x_s.  For
    sublayer q (mixer, then feed-forward) with vectors in_q, out_q and a matrix mix_q ([from, to]):

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + mult * out_q[t] * y

    for all t at once from the old streams.  ``streams`` 0 is the plain residual x <- x + mult * y: one
    stream and no tensors.  The tensors of sublayer q are ``prefix + connection_prefixes[q] + "in" | "out" | "mix"``."""
    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    streams: int = 0
    residual_mult: float = 1.0
    block: str = "hyper"
    mixer_prefix: str = "mix."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "norm1"
    feed_forward_norm_prefix: str = "norm2"
    connection_prefixes: Tuple[str, str] = ("hc1.", "hc2.")


@dataclass(frozen=True)
class PostNormLayerSpec:
    """One layer whose sublayers read the residual itself and whose norms stand behind them:

        x <- x + mult * scale_1 * norm_1(mixer(x));    x <- x + mult * scale_2 * norm_2(feed_forward(x))

    ``scale_q``: a learned vector per sublayer (tensor ``prefix + scale_names[q]``; None: no such vector).
    ``feed_forward`` and ``feed_forward_norm`` None: the layer is its mixer sublayer alone."""
    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    residual_mult: float = 1.0
    scale_names: Optional[Tuple[str, str]] = ("ls1", "ls2")
    block: str = "postnorm"
    mixer_prefix: str = "mix."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "norm1"
    feed_forward_norm_prefix: str = "norm2"


@dataclass(frozen=True)
class ReinjectSpec:
    """What happens to the residual where a pass through repeated layers begins: with the embedding output x0,

        x <- W [x; x0] + steps[index]

    W: the tensor ``weight`` ([hidden, 2 hidden], the residual's columns first); ``steps``: a tensor
    [passes, hidden] of one vector per pass.  The product's inputs are in the activation dtype, its sums and the
    new residual float32."""
    hidden: int
    passes: int
    index: int
    weight: str = "loop.in"
    steps: str = "loop.step"
    kind: str = "reinject"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers``; a layer may appear in several entries (its weights are
    then used more than once, each run with a cache plane of its own).  ``cache_of`` names the
    schedule position whose cache plane this run reads instead of writing one of its own
    (None: own plane).  ``enter``: the spec of a *junction* part (registry category ``junction``) that
    rewrites the residual right before this run (``ReinjectSpec``), or None.
    """
    layer: int
    cache_of: Optional[int] = None
    enter: Optional[object] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    """``scale`` multiplies every embedding row as it enters the float32 residual."""
    name: str
    vocab: int
    hidden: int
    scale: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """Output projection hidden -> vocab.  If the checkpoint has no tensor ``name`` the head is
    tied to ``tied_to`` (qwen3/chat.go:55-65 decides by tensor presence, never by a flag)."""
    name: str
    vocab: int
    hidden: int
    tied_to: Optional[str] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    final_norm_name: str
    head: HeadSpec
    streams: int = 1      # copies of the residual the blocks keep (hyper-connections); the final norm reads their sum

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("model spec: no layers")
        if not self.schedule:
            raise ValueError("model spec: empty schedule")
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"model spec: schedule[{pos}] names layer {e.layer}, "
                                 f"there are {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < pos:
                    raise ValueError(f"model spec: schedule[{pos}] reads the cache of position "
                                     f"{e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"model spec: schedule[{pos}] reads the cache of position "
                                     f"{e.cache_of}, which has no cache of its own")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))
