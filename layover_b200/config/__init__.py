from .base import (
    DTYPE_BYTES,
    Architecture,
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    supported_architectures,
    unregister_architecture,
)
from .qwen3 import PRESETS, Qwen3Config
from .qwen3 import preset as _qwen3_preset
from .kirenex import KIRENEX_PRESETS, KirenexConfig
from .limazen import LIMAZEN_PRESETS, LimazenConfig
from .topidra import TOPIDRA_PRESETS, TopidraConfig
from .vopozen import VOPOZEN_PRESETS, VopozenConfig


def preset(name: str, **overrides):
    """The configuration of a named shape, of whichever architecture has that name."""
    if name in VOPOZEN_PRESETS:
        return VopozenConfig(**{**VOPOZEN_PRESETS[name], **overrides})
    if name in KIRENEX_PRESETS:
        return KirenexConfig(**{**KIRENEX_PRESETS[name], **overrides})
    if name in LIMAZEN_PRESETS:
        return LimazenConfig(**{**LIMAZEN_PRESETS[name], **overrides})
    if name in TOPIDRA_PRESETS:
        return TopidraConfig(**{**TOPIDRA_PRESETS[name], **overrides})
    if name not in PRESETS:
        raise ValueError(f"unknown preset {name!r}; known: {sorted(PRESETS) + sorted(TOPIDRA_PRESETS) + sorted(LIMAZEN_PRESETS) + sorted(KIRENEX_PRESETS) + sorted(VOPOZEN_PRESETS)}")
    return _qwen3_preset(name, **overrides)


__all__ = [
    "DTYPE_BYTES", "Architecture", "load_config", "read_config_json", "register_architecture",
    "resolve_architecture", "supported_architectures", "unregister_architecture",
    "PRESETS", "Qwen3Config", "preset", "TOPIDRA_PRESETS", "TopidraConfig", "LIMAZEN_PRESETS", "LimazenConfig", "KIRENEX_PRESETS", "KirenexConfig", "VOPOZEN_PRESETS", "VopozenConfig",
]
