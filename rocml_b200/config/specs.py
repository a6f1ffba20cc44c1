"""Architecture-neutral description of a decoder: what each layer is made of.

An architecture's typed configuration (for example ``Qwen3Config``) is turned
into a ``ModelSpec``.  Everything below the configuration (parts, cache, engine)
reads only these specs, so no part knows which model it sits in, and layers of
one model may differ from one another.

A spec names a *kind* (a string looked up in the part registries of
``rocml_b200.parts``) and carries that kind's sizes and constants.  Kinds that a
test or a user registers later need no change here: ``MixerSpec`` and
``FeedForwardSpec`` keep free-form ``params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _frozen_params(params: Optional[Mapping[str, Any]]) -> Tuple[Tuple[str, Any], ...]:
    """Parameters as a sorted tuple of pairs; a mapping among the values (``names``) is frozen the same way."""
    return tuple(sorted((k, _frozen_params(v) if isinstance(v, Mapping) else v) for k, v in (params or {}).items()))


def tensor_names(params: Mapping[str, Any], defaults: Mapping[str, str]) -> dict:
    """A part's tensor-name stems: ``defaults`` (role -> stem) overridden by the spec's ``names``
    parameter.  A role the part does not know is an error: it would silently name nothing."""
    given = dict(params.get("names") or ())
    unknown = sorted(set(given) - set(defaults))
    if unknown:
        raise ValueError(f"names for unknown tensors {unknown}; this part has {sorted(defaults)}")
    return {**defaults, **given}


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.  kind "rmsnorm": x * rsqrt(mean(x^2) + eps) * (w + weight_offset);
    ``weight_offset`` 1 is a weight that the files store around zero."""

    kind: str = "rmsnorm"
    eps: float = 1e-6
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope_neox": rotate-half rotary embedding over the first ``rot_dim``
    dimensions of every head with base ``theta``; kind "rope_pairs": the same with
    neighbouring entries (2i, 2i + 1) as pairs; both take the parameter ``scaling``
    ({factor, low, high, original}: long wavelengths stretched) or ``ramp_scaling``
    ({factor, original, fast, slow}: frequencies blended between f and f / factor along a ramp over
    the pair index, and cosines and sines times 0.1 ln(factor) + 1); kind "none": nothing.
    As a model's ``input_position`` (added to the embedding output, not applied inside a mixer):
    kind "sinusoid": entry 2i of the vector is sin(pos * theta^(-2i / width)), entry 2i + 1 the cosine.
    """

    kind: str = "rope_neox"
    theta: float = 1e6
    rot_dim: Optional[int] = None  # None: the whole head
    params_items: Tuple[Tuple[str, Any], ...] = ()

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class MixerSpec:
    """The token mixer of a layer.  kind "attention" is grouped-query softmax attention.

    Attention params: n_heads, n_kv_heads, head_dim, bias (q/k/v/o biases),
    qk_norm (per-head RMSNorm of q and k before the position encoding),
    qk_norm_eps, window (None: every earlier key; n: the last n keys, the
    query's own position included), scale (None: 1/sqrt(head_dim)),
    names (the tensor-name stems under the layer's mixer prefix, by role:
    q, k, v, o, q_norm, k_norm, gate; default q_proj, k_proj, v_proj, o_proj,
    q_norm, k_norm, gate_proj), v_head_dim (the value heads' size when it is not
    head_dim), chunk (a query sees the earlier keys of its own block of that many
    positions, blocks counted from position 0; not together with window), gated (head
    n's result is multiplied by sigmoid(Wgate x)_n before the output projection; "per_value": the
    gate has a number for every value of every head), bias as a list of the roles that have
    one (["q", "k", "v"]) instead of all or none, keep_first (with a window: the keys at positions
    below it stay visible to every later query), sink (a score s: every row's softmax denominator
    has one more term exp(s) that brings no value), qk_unit_norm (queries and keys divided by their
    root mean square over the head, without a weight, after the position encoding; eps is
    qk_norm_eps), value_mix ("source": this layer's values as projected are kept for the step;
    "mix": what is cached and read is (1 - lambda) v + lambda v_source, lambda the layer's scalar
    tensor of role value_mix, v_source the values of the same token in the step's source layer).
    """

    kind: str
    params_items: Tuple[Tuple[str, Any], ...] = ()
    position: PositionSpec = PositionSpec(kind="none")

    # Kind "linear_attention" (a decayed running sum S = d_h S + k v^T per head instead of a softmax; state of fixed
    # size a sequence): n_heads, head_dim, v_head_dim, decay (one number a head), qk_activation and v_activation
    # ("none" | "silu"), k_scale, out_norm ("per_head" | "all_heads") with out_norm_eps and out_norm_weight (bool),
    # gate_activation ("silu" | "sigmoid"), names (roles q, k, v, gate, o, out_norm).
    # Kind "latent_attention" (keys and values unfolded from one cached latent vector a token): n_heads, head_dim
    # (queries and keys), v_head_dim, kv_rank, latent_norm_eps, window, scale, gated (a sigmoid gate per head on the
    # attention's output, read from the mixer's input), names (roles q, down, latent_norm, up_k, up_v, gate, o).

    @staticmethod
    def make(kind: str, position: Optional[PositionSpec] = None, **params) -> "MixerSpec":
        return MixerSpec(kind, _frozen_params(params), position or PositionSpec(kind="none"))

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class FeedForwardSpec:
    """The feed-forward of a layer.  kind "gated_mlp": down(act(gate(x)) * up(x)).

    gated_mlp params: intermediate, activation ("silu"), bias, names (the
    tensor-name stems under the layer's feed-forward prefix, by role: gate,
    up, down; default gate_proj, up_proj, down_proj).

    routed_mlp (a router and ``experts`` small gated feed-forwards, ``top`` of them a token) params: experts, top,
    intermediate, activation ("silu" or "clamped_swish" with ``limit`` and ``alpha``), score ("sigmoid"),
    choice_bias (a per-expert vector added to the scores for the choice only), renormalize, names (roles router,
    choice_bias, expert (a pattern with {e}), gate, up, down).
    """

    kind: str
    params_items: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def make(kind: str, **params) -> "FeedForwardSpec":
        return FeedForwardSpec(kind, _frozen_params(params))

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: two norms, a mixer and a feed-forward in a named arrangement.

    arrangement "pre_norm": x += mixer(norm1(x)); x += ff(norm2(x)).
    arrangement "parallel": x += mixer(norm1(x)) + ff(norm1(x)); "parallel_two_norms": x += mixer(norm1(x)) +
    ff(norm2(x)), both norms of the same x.
    arrangement "sandwich_norm": x += post1(mixer(norm1(x))); x += post2(ff(norm2(x))), with the two
    post norms given by ``mixer_post_norm`` and ``ff_post_norm``; ``feed_forward`` None leaves the second half out.
    arrangement "post_norm": x <- norm1(alpha x + g1 * mixer(h)); x <- norm2(alpha x + g2 * ff(x)): the norm follows the
    sum and the sublayers read the stream itself.  Its constants are ``arrangement_items``: alpha (default 1),
    layer_scale (the vectors g1, g2 exist; default False), token_shift (h_t = x_t + (x_(t-1) - x_t) * mu with a vector mu,
    the row before kept per sequence; default False: h = x), names (roles mixer_scale, ff_scale, shift).
    ``prefix`` is the layer's tensor-name prefix in the weight files; under it the four parts'
    tensors are named ``<prefix>.<mixer_norm_name>.weight``, ``<prefix>.<mixer_name><stem>...``,
    ``<prefix>.<ff_norm_name>.weight`` and ``<prefix>.<ff_name><stem>...`` (the defaults are the
    names of Hugging Face's Qwen3 checkpoints; another architecture gives its own).
    """

    prefix: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    ff_norm: NormSpec
    arrangement: str = "pre_norm"
    mixer_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn."
    ff_norm_name: str = "post_attention_layernorm"
    ff_name: str = "mlp."
    mixer_post_norm: Optional[NormSpec] = None
    ff_post_norm: Optional[NormSpec] = None
    mixer_post_norm_name: str = "post_mixer_norm"
    ff_post_norm_name: str = "post_ff_norm"
    arrangement_items: Tuple[Tuple[str, Any], ...] = ()     # the arrangement's own constants (see above)

    @property
    def arrangement_params(self) -> dict:
        return {k: (dict(v) if isinstance(v, tuple) and v and isinstance(v[0], tuple) else v) for k, v in self.arrangement_items}


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers``.

    ``reads_cache_of`` names an earlier schedule entry whose cache this run
    reads instead of keeping its own (it then writes nothing).  Every other
    entry keeps a cache of its own, also when its layer runs more than once.

    Before the run, two things may be added to the residual stream, in this
    order: the embedding output (``add_input``), and row ``add_row[1]`` of the
    [``add_row[2]``, hidden] tensor named ``add_row[0]``.
    """

    layer: int
    reads_cache_of: Optional[int] = None
    add_input: bool = False
    add_row: Optional[Tuple[str, int, int]] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, head."""

    architecture: str
    hidden: int
    vocab: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    stop_tokens: Tuple[int, ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = field(default=())
    embedding_scale: float = 1.0                       # the gathered rows are multiplied by it
    input_position: Optional[PositionSpec] = None      # a position vector added to the embedding output
    logit_scale: float = 1.0                           # the head's result is multiplied by it
    weight_suffix: str = ".weight"                     # what the files append to a part's tensor-name stem
    bias_suffix: str = ".bias"                         # the same for a part's '<stem>.bias'
    embedding_norm: Optional[NormSpec] = None          # a norm of the embedding output, before the first layer
    embedding_norm_name: str = "model.embed_norm.weight"

    def __post_init__(self):
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer}, model has {n}")
            if e.reads_cache_of is not None and not 0 <= e.reads_cache_of < i:
                raise ValueError(
                    f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                    "which must be an earlier entry"
                )
