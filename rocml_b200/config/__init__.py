"""Typed configurations, the architecture registry and the catalog of short names."""
from .specs import (
    FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
)
from .qwen3 import Qwen3Config, ARCHITECTURE as QWEN3_ARCHITECTURE
from .pipilix import PipilixConfig, ARCHITECTURE as PIPILIX_ARCHITECTURE
from .zokelorn import ZokelornConfig, ARCHITECTURE as ZOKELORN_ARCHITECTURE
from .safesun import SafesunConfig, ARCHITECTURE as SAFESUN_ARCHITECTURE
from .tibenex import TibenexConfig, ARCHITECTURE as TIBENEX_ARCHITECTURE
from .registry import (
    CATALOG, CatalogEntry, ResolvedModel, SamplingPreset, checkpoint_dir, config_from_dict,
    load_config, load_model_spec, register_architecture, registered_architectures, resolve,
)

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config.from_dict)
register_architecture(PIPILIX_ARCHITECTURE, PipilixConfig.from_dict)
register_architecture(ZOKELORN_ARCHITECTURE, ZokelornConfig.from_dict)
register_architecture(SAFESUN_ARCHITECTURE, SafesunConfig.from_dict)
register_architecture(TIBENEX_ARCHITECTURE, TibenexConfig.from_dict)

__all__ = [
    "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
    "ScheduleEntry", "Qwen3Config", "QWEN3_ARCHITECTURE", "PipilixConfig", "PIPILIX_ARCHITECTURE", "ZokelornConfig", "ZOKELORN_ARCHITECTURE",
    "SafesunConfig", "SAFESUN_ARCHITECTURE", "TibenexConfig", "TIBENEX_ARCHITECTURE", "CATALOG", "CatalogEntry",
    "ResolvedModel", "SamplingPreset", "checkpoint_dir", "config_from_dict", "load_config",
    "load_model_spec", "register_architecture", "registered_architectures", "resolve",
]
