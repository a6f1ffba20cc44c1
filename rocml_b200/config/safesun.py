"""Typed configuration of the Safesun decoder, read from config.json.

A Safesun model is an embedding followed by a norm, a list of layers that each name their mixer with its
own sizes and an optional dense gated feed-forward (silu), a final norm and a head that is the embedding
table.  Every layer is parallel with two norms of the same input, one for the mixer and one for the
feed-forward; every norm's weight is stored around zero (the factor is 1 + w).  Two mixers, both grouped-query
softmax attention under a sliding window that also keeps the first positions visible, with rotate-half
rotation of part of every head, a sigmoid gate for every value of the result, and values that later layers
may blend with those of the first layer that takes part:

* ``attention``: per-head RMS norm of queries and keys with a weight, before the rotation; the rotation's
  frequencies may be blended along a ramp (factor, original, fast, slow) with a magnitude on cosines and sines;
  an ordinary softmax.
* ``attention_2``: biases on the q, k and v projections; queries and keys divided by their root mean square
  after the rotation, without a weight; a softmax whose denominator has one more term of score 0.

Keys read (every size and every constant that differs between models comes from here)::

    architecture        "Safesun"
    vocab, width
    norm.eps
    layers[i].type      "attention" | "attention_2"
    layers[i].mixer     heads, kv_heads, dim, vdim, scale, mask: {size, keep_first}, v_mix,
                        rot: {base, dims, scaling: {factor, original, fast, slow} (optional)}
    layers[i].mlp       null | {kind: "dense", ff}

Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<q|k|v|g|o>``,
``l<i>.mix.<q|k|v>.b`` (attention_2), ``l<i>.mix.<q|k>.norm`` (attention), ``l<i>.mix.vmix`` (layers that mix
values), ``l<i>.mlp.<gate|up|down>``, ``final.norm``; no ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .pipilix import _get, _int, _num
from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, _frozen_params

ARCHITECTURE = "Safesun"

# Constants the design fixes.
SINK_SCORE = 0.0               # attention_2: the score of the term that the softmax's denominator has beside the keys
NORM_WEIGHT_OFFSET = 1.0       # norms of the stream multiply by 1 + w
MAX_CONTEXT = 1 << 20          # the design names no longest sequence: positions are plain integers

_MIXERS = ("attention", "attention_2")


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None     # factor, original, fast, slow

    @staticmethod
    def from_dict(d, where) -> "RotationConfig":
        sc = d.get("scaling") if isinstance(d, Mapping) else None
        scaling = None
        if sc is not None:
            w = where + "scaling."
            scaling = (_num(sc, "factor", w), _num(sc, "original", w), _num(sc, "fast", w), _num(sc, "slow", w))
            if not (scaling[0] > 0 and scaling[1] > 0 and scaling[2] > 0 and scaling[3] > 0):
                raise ConfigError(f"config.json: {w}factor, original, fast and slow must be positive")
        cfg = RotationConfig(_num(d, "base", where), _int(d, "dims", where, 0), scaling)
        if cfg.dims % 2:
            raise ConfigError(f"config.json: {where}dims must be even, found {cfg.dims}")
        if not cfg.base > 0 or (scaling is not None and cfg.base == 1.0):
            raise ConfigError(f"config.json: {where}base must be positive (and not 1 with scaling), found {cfg.base}")
        return cfg

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]              # mask.size: a query sees the last `window` keys, its own included
    keep_first: int                    # mask.keep_first: and the keys at positions below this
    rot: Optional[RotationConfig]
    v_mix: bool

    @staticmethod
    def from_dict(d, where) -> "AttentionConfig":
        mask = d.get("mask") if isinstance(d, Mapping) else None
        rot = d.get("rot") if isinstance(d, Mapping) else None
        v_mix = d.get("v_mix", False) if isinstance(d, Mapping) else False
        if not isinstance(v_mix, bool):
            raise ConfigError(f"config.json: {where}v_mix must be true or false, found {v_mix!r}")
        keep = 0
        if mask is not None and mask.get("keep_first") is not None:
            keep = _int(mask, "keep_first", where + "mask.", 0)
        cfg = AttentionConfig(
            heads=_int(d, "heads", where), kv_heads=_int(d, "kv_heads", where), dim=_int(d, "dim", where),
            vdim=_int(d, "vdim", where), scale=_num(d, "scale", where),
            window=None if mask is None else _int(mask, "size", where + "mask."), keep_first=keep,
            rot=None if rot is None else RotationConfig.from_dict(rot, where + "rot."), v_mix=v_mix)
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}heads {cfg.heads} is no multiple of kv_heads {cfg.kv_heads}")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise ConfigError(f"config.json: {where}rot.dims {cfg.rot.dims} exceeds dim {cfg.dim}")
        return cfg

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "v_mix": self.v_mix}
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class SafesunLayer:
    mixer_type: str                    # "attention" or "attention_2"
    mixer: AttentionConfig
    ff: Optional[int]                  # the dense feed-forward's inner width; None: the layer has none


@dataclass(frozen=True)
class SafesunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SafesunLayer, ...]

    def __post_init__(self):
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        mixing = [L.mixer for L in self.layers if L.mixer.v_mix]
        if len({(m.kv_heads, m.vdim) for m in mixing}) > 1:
            raise ConfigError("config.json: the layers that say v_mix blend their values with the first such layer's, "
                              "so they must agree in kv_heads and vdim")

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "SafesunConfig":
        layers = _get(d, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("config.json: 'layers' must be a list")
        out = []
        for i, L in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is unknown (known: {', '.join(_MIXERS)})")
            mixer = AttentionConfig.from_dict(_get(L, "mixer", where), where + "mixer.")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if _get(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is unknown (known: dense)")
                ff = _int(mlp, "ff", where + "mlp.")
            out.append(SafesunLayer(kind, mixer, ff))
        return SafesunConfig(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                             norm_eps=_num(_get(d, "norm", ""), "eps", "norm."), layers=tuple(out))

    def to_dict(self) -> dict:
        return {
            "architecture": ARCHITECTURE,
            "layers": [{"type": L.mixer_type, "mixer": L.mixer.to_dict(),
                        "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}} for L in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    # ---- the architecture, spelled as parts ------------------------------------------------------
    def _mixer_spec(self, L: SafesunLayer, value_mix: Optional[str]) -> MixerSpec:
        m = L.mixer
        position = None
        if m.rot is not None and m.rot.dims > 0:
            params = {}
            if m.rot.scaling is not None:
                params["ramp_scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
            position = PositionSpec("rope_neox", theta=m.rot.base, rot_dim=m.rot.dims, params_items=_frozen_params(params))
        second = L.mixer_type == "attention_2"
        return MixerSpec.make(
            "attention", position, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
            scale=m.scale, window=m.window, keep_first=m.keep_first if m.window is not None else 0,
            gated="per_value", bias=("q", "k", "v") if second else False,
            qk_norm=not second, qk_norm_eps=self.norm_eps, qk_unit_norm=second, sink=SINK_SCORE if second else None,
            value_mix=value_mix,
            names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_norm": "q.norm", "k_norm": "k.norm",
                   "value_mix": "vmix"})

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.norm_eps, NORM_WEIGHT_OFFSET)
        layers = []
        source_seen = False
        for i, L in enumerate(self.layers):
            value_mix = None
            if L.mixer.v_mix:
                value_mix = "mix" if source_seen else "source"
                source_seen = True
            ff = None if L.ff is None else FeedForwardSpec.make(
                "gated_mlp", intermediate=L.ff, activation="silu", bias=False, names={"gate": "gate", "up": "up", "down": "down"})
            layers.append(LayerSpec(
                prefix=f"l{i}", mixer=self._mixer_spec(L, value_mix), feed_forward=ff, mixer_norm=norm, ff_norm=norm,
                arrangement="parallel_two_norms", mixer_norm_name="norm1", ff_norm_name="norm2", mixer_name="mix.",
                ff_name="mlp."))
        return ModelSpec(
            architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_position=MAX_CONTEXT, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm, tie_embeddings=True,
            embedding_name="embed.weight", final_norm_name="final.norm.weight", head_name="head.weight", weight_suffix="",
            bias_suffix=".b", embedding_norm=norm, embedding_norm_name="embed.norm.weight")
