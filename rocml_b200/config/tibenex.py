"""Typed configuration of the Tibenex decoder, read from config.json.

A Tibenex model is an embedding times a constant, a list of layers that each name their mixer with its own
sizes and an optional dense gated feed-forward (silu), a final norm and a head of its own.  A layer
normalises AFTER the sum: x <- norm1(alpha x + g1 * mixer(h)), x <- norm2(alpha x + g2 * ff(x)), with a
vector g per sublayer (the layer's scale) and h the layer's input blended with the token before it,
h_t = x_t + (x_(t-1) - x_t) * mu.  Three mixers:

* ``latent_attention``: queries through a latent of their own (normalised), keys and values unfolded from one
  cached latent a token, plus one rotated key part shared by all heads; rotate-half rotation whose
  frequencies are blended along a ramp (factor, original, fast, slow) with a magnitude on cosines and sines;
  a sigmoid gate per head.
* ``attention``: grouped-query softmax attention with an RMS norm over the whole q and the whole k
  projection, rotation of neighbouring pairs, a temperature per head on the scores, and the heads'
  weights mixed by a matrix after the softmax.
* ``mamba2``: a state-space mixer: a short causal convolution over x, B and C, a step size per token and
  head, the recurrence S = exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x, a silu gate, a norm in equal parts.

Keys read (every size and every constant that differs between models comes from here)::

    architecture        "Tibenex"
    vocab, width, postln_alpha
    embedding.scale, norm.eps
    layers[i].type      "latent_attention" | "attention" | "mamba2"
    layers[i].mixer     latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                          rot: {base, dims, scaling: {factor, original, fast, slow} (optional)}
                        attention: heads, kv_heads, dim, vdim, scale, rot: {base, dims}
                        mamba2: heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp       null | {kind: "dense", ff}

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.shift``,
``l<i>.mix.<dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o>``, ``l<i>.mix.<q|k|v|q.norm|k.norm|talk|temp|o>``,
``l<i>.mix.<in|conv|conv.b|dt_bias|A_log|D|norm|o>``, ``l<i>.mlp.<gate|up|down>``, ``final.norm``, ``head``;
no ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import ConfigError
from .pipilix import _get, _int, _num
from .safesun import RotationConfig
from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, _frozen_params

ARCHITECTURE = "Tibenex"

MAX_CONTEXT = 1 << 20          # the design names no longest sequence: positions are plain integers

_MIXERS = ("latent_attention", "attention", "mamba2")


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int                # unrotated query/key entries a head
    rot_dim: int            # rotated entries a head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Optional[RotationConfig]

    @staticmethod
    def from_dict(d, where) -> "LatentConfig":
        rot = d.get("rot") if isinstance(d, Mapping) else None
        rot_dim = _int(d, "rot_dim", where, 0)
        if isinstance(rot, Mapping) and rot.get("dims") is None:
            rot = {**rot, "dims": rot_dim}          # the rotated vector is the rot_dim part
        cfg = LatentConfig(heads=_int(d, "heads", where), dim=_int(d, "dim", where, 0), rot_dim=rot_dim, vdim=_int(d, "vdim", where),
                           kv_rank=_int(d, "kv_rank", where), q_rank=_int(d, "q_rank", where), scale=_num(d, "scale", where),
                           rot=None if rot is None else RotationConfig.from_dict(rot, where + "rot."))
        if cfg.rot_dim % 2:
            raise ConfigError(f"config.json: {where}rot_dim must be even, found {cfg.rot_dim}")
        if cfg.rot_dim and cfg.rot is None:
            raise ConfigError(f"config.json: {where}rot_dim is {cfg.rot_dim} but {where}rot is absent")
        if cfg.dim + cfg.rot_dim == 0:
            raise ConfigError(f"config.json: {where}dim and rot_dim cannot both be 0")
        return cfg

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "q_rank": self.q_rank, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]

    @staticmethod
    def from_dict(d, where) -> "TalkingAttentionConfig":
        rot = d.get("rot") if isinstance(d, Mapping) else None
        cfg = TalkingAttentionConfig(heads=_int(d, "heads", where), kv_heads=_int(d, "kv_heads", where), dim=_int(d, "dim", where),
                                     vdim=_int(d, "vdim", where), scale=_num(d, "scale", where),
                                     rot=None if rot is None else RotationConfig.from_dict(rot, where + "rot."))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}heads {cfg.heads} is no multiple of kv_heads {cfg.kv_heads}")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise ConfigError(f"config.json: {where}rot.dims {cfg.rot.dims} exceeds dim {cfg.dim}")
        if cfg.rot is not None and cfg.rot.scaling is not None:
            raise ConfigError(f"config.json: {where}rot.scaling is not part of this mixer")
        return cfg

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int               # columns of a head's state (the head's share of x)
    state: int              # rows of a head's state (the size of B and C)
    groups: int             # B and C are shared by heads / groups heads
    conv: int               # taps of the causal convolution
    norm_groups: int        # the gated result is normalised in this many equal parts

    @staticmethod
    def from_dict(d, where) -> "StateSpaceConfig":
        cfg = StateSpaceConfig(heads=_int(d, "heads", where), vdim=_int(d, "vdim", where), state=_int(d, "state", where),
                               groups=_int(d, "groups", where), conv=_int(d, "conv", where), norm_groups=_int(d, "norm_groups", where))
        if cfg.heads % cfg.groups:
            raise ConfigError(f"config.json: {where}heads {cfg.heads} is no multiple of groups {cfg.groups}")
        if (cfg.heads * cfg.vdim) % cfg.norm_groups:
            raise ConfigError(f"config.json: {where}norm_groups {cfg.norm_groups} does not divide heads * vdim = {cfg.heads * cfg.vdim}")
        return cfg

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


_MIXER_CONFIGS = {"latent_attention": LatentConfig, "attention": TalkingAttentionConfig, "mamba2": StateSpaceConfig}


@dataclass(frozen=True)
class TibenexLayer:
    mixer_type: str
    mixer: Union[LatentConfig, TalkingAttentionConfig, StateSpaceConfig]
    ff: Optional[int]                  # the dense feed-forward's inner width; None: the layer has none


@dataclass(frozen=True)
class TibenexConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    embedding_scale: float
    layers: Tuple[TibenexLayer, ...]

    def __post_init__(self):
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "TibenexConfig":
        layers = _get(d, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("config.json: 'layers' must be a list")
        out = []
        for i, L in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is unknown (known: {', '.join(_MIXERS)})")
            mixer = _MIXER_CONFIGS[kind].from_dict(_get(L, "mixer", where), where + "mixer.")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if _get(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is unknown (known: dense)")
                ff = _int(mlp, "ff", where + "mlp.")
            out.append(TibenexLayer(kind, mixer, ff))
        return TibenexConfig(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                             norm_eps=_num(_get(d, "norm", ""), "eps", "norm."), postln_alpha=_num(d, "postln_alpha", ""),
                             embedding_scale=_num(_get(d, "embedding", ""), "scale", "embedding."), layers=tuple(out))

    def to_dict(self) -> dict:
        return {
            "architecture": ARCHITECTURE,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": L.mixer_type, "mixer": L.mixer.to_dict(),
                        "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}} for L in self.layers],
            "norm": {"eps": self.norm_eps},
            "postln_alpha": self.postln_alpha,
            "vocab": self.vocab,
            "width": self.width,
        }

    # ---- the architecture, spelled as parts ------------------------------------------------------
    def _position(self, rot: Optional[RotationConfig], dims: int, kind: str) -> Optional[PositionSpec]:
        if rot is None or dims <= 0:
            return None
        params = {}
        if rot.scaling is not None:
            params["ramp_scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot.scaling))
        return PositionSpec(kind, theta=rot.base, rot_dim=dims, params_items=_frozen_params(params))

    def _mixer_spec(self, L: TibenexLayer) -> MixerSpec:
        m = L.mixer
        if L.mixer_type == "latent_attention":
            # the rotated vector is the rot_dim part: the rotation's frequencies are those of a head of rot_dim entries
            return MixerSpec.make(
                "latent_attention", self._position(m.rot, m.rot_dim, "rope_neox"), n_heads=m.heads, head_dim=m.dim,
                rot_head_dim=m.rot_dim, v_head_dim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank, latent_norm_eps=self.norm_eps,
                scale=m.scale, gated=True,
                names={"q_down": "dq", "q_latent_norm": "dq.norm", "q": "uq", "down": "dkv", "latent_norm": "dkv.norm",
                       "up_k": "uk", "up_v": "uv", "gate": "g", "o": "o"})
        if L.mixer_type == "attention":
            return MixerSpec.make(
                "attention", self._position(m.rot, m.rot.dims if m.rot is not None else 0, "rope_pairs"), n_heads=m.heads,
                n_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim, scale=m.scale, qk_norm="whole",
                qk_norm_eps=self.norm_eps, head_temperature=True, talking_heads=True,
                names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "talk": "talk",
                       "temperature": "temp"})
        return MixerSpec.make(
            "state_space", None, n_heads=m.heads, head_dim=m.vdim, state=m.state, groups=m.groups, conv_taps=m.conv,
            norm_groups=m.norm_groups, norm_eps=self.norm_eps,
            names={"in": "in", "conv": "conv", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D", "norm": "norm", "o": "o"})

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.norm_eps)
        layers = []
        for i, L in enumerate(self.layers):
            ff = None if L.ff is None else FeedForwardSpec.make(
                "gated_mlp", intermediate=L.ff, activation="silu", bias=False, names={"gate": "gate", "up": "up", "down": "down"})
            layers.append(LayerSpec(
                prefix=f"l{i}", mixer=self._mixer_spec(L), feed_forward=ff, mixer_norm=norm, ff_norm=norm,
                arrangement="post_norm", mixer_norm_name="norm1", ff_norm_name="norm2", mixer_name="mix.", ff_name="mlp.",
                arrangement_items=_frozen_params({"alpha": self.postln_alpha, "layer_scale": True, "token_shift": True,
                                                  "names": {"mixer_scale": "ls1", "ff_scale": "ls2", "shift": "shift"}})))
        return ModelSpec(
            architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_position=MAX_CONTEXT, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm, tie_embeddings=False,
            embedding_name="embed.weight", final_norm_name="final.norm.weight", head_name="head.weight", weight_suffix="",
            bias_suffix=".b", embedding_scale=self.embedding_scale)
